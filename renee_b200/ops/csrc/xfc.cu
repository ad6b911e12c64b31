// Extreme-classifier (XFC) step kernels for sm_100a: three tcgen05/TMEM GEMMs with fused epilogues.
//
//   logits_grad  Gt[l, b]  = sigmoid(sum_d W[l,d] X[b,d]) - Y[l,b]     (A = W K-major, B = X K-major)
//                 epilogue: sigmoid in registers, fp16 store, positives patched from a label-sorted COO
//                 list by binary search, optional sparse-BCE loss partials.  Logits never reach HBM.
//   dx           dX[b, d] += scale * sum_l Gt[l,b] W[l,d]              (A = Gt MN-major, B = W MN-major)
//                 split over label blocks, fp32 accumulation in TMEM, vector red.add into dX.
//   dw_sgd       dW[l, d]  = sum_b Gt[l,b] X[b,d]                      (A = Gt K-major, B = X MN-major)
//                 epilogue: g = dW + wd W; M = mo M + g; W -= lr M on the fp16 W / M tiles (dW never
//                 stored).
//
// They replace, in the reference: torch.matmul/addmm through cuBLAS (dl_base.py:572, 606-608, 625-633),
// the CUTLASS Volta sigmoid-GEMM / dW GEMM of xfc_gemm_kernel.cu:59-150, torch.sigmoid + index_put_
// (dl_base.py:593-594), the sampled loss reductions (dl_base.py:579-583) and apex FusedSGD
// (dl_base.py:343).
//
// Structure of every kernel: 192 threads; warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (one TMEM lane quarter each).  4-stage smem ring, 128x{<=256}x64 tiles,
// UMMA 128xNx16.  All waits are bounded (see tc.cuh).
#include "peer.cuh"

namespace rb {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kStages = 4;
constexpr int kABytes = kBM * kBK * 2;          // 16 KB
constexpr int kBBytesMax = 256 * kBK * 2;       // 32 KB
constexpr int kStageBytes = kABytes + kBBytesMax;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr int kThreads = 192;
constexpr int kTmemCols = 256;

enum Mode : int { MODE_LOGITS = 0, MODE_DX = 1, MODE_DW = 2, MODE_RAW = 3 };

struct GemmParams {
  int M;             // valid output rows   (labels for LOGITS/DW/RAW, batch rows for DX)
  int N;             // valid output cols   (batch rows for LOGITS/RAW, D for DX/DW)
  int BN;            // N tile (multiple of 16, <= 256)
  int kb_total;      // number of 64-wide k blocks
  int kb_per_split;  // k blocks handled by one blockIdx.z
  int* status;
  // LOGITS / RAW
  __half* Gt; int ldG;
  const int* pos_rows; const int* pos_labels; const int* nnz_ptr; int label0;
  float* loss_acc;
  // DX
  float* dX; int ldX; const float* hp;
  // DW
  __half* W; __half* Mom; int ldW; float mo; float wd;
  float* Zout;       // RAW: fp32 logits, batch-major Zt[N, ldG] (top-k path)
  // multi-GPU fusion (null / 0 when unused)
  const uint32_t* wait_flags; int wait_n; StepTag tag;   // LOGITS: X rows of every rank have landed
  unsigned* done_counter; PeerPtrs peer_flags; int n_peers; int flag_index;   // DX: last CTA raises "partial complete"
  int stochastic_round;   // DW (TMA kernel): round the updated weights to fp16 stochastically
};

__device__ __forceinline__ int lower_bound_i32(const int* a, int n, int key) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
xfc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  constexpr bool A_MN = (MODE == MODE_DX);
  constexpr bool B_MN = (MODE == MODE_DX || MODE == MODE_DW);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_full_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kBM;
  const int n0 = blockIdx.y * p.BN;
  const int kb0 = blockIdx.z * p.kb_per_split;
  const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
  const bool has_work = kb1 > kb0;
  const uint32_t b_bytes = (uint32_t)p.BN * kBK * 2;

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
    for (int s = 0; s < kStages; ++s) { tc::mbar_init(full_bar + s, 1); tc::mbar_init(empty_bar + s, 1); }
    tc::mbar_init(tmem_full_bar, 1);
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_ptr_smem, kTmemCols);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  bool aborted = false;

  if (warp == 0 && lane == 0 && has_work) {
    // ---------------- TMA producer
    if (MODE == MODE_LOGITS && p.wait_flags != nullptr) {
      // all-gather prologue: every rank has pushed its rows of X into this GPU's buffer and raised its
      // flag; the loads below go through the async proxy, hence the proxy fence after the acquire
      const uint32_t want = p.tag.value();
      for (int q = 0; q < p.wait_n; ++q)
        if (!wait_flag(p.wait_flags + q, want, p.status, 100 + q)) aborted = true;
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    for (int kb = kb0, it = 0; kb < kb1 && !aborted; ++kb, ++it) {
      const int s = it % kStages;
      const uint32_t ph = (it / kStages) & 1;
      if (!tc::mbar_wait(empty_bar + s, ph ^ 1, aborted, p.status, tc::SITE_EMPTY, kb)) break;
      uint8_t* sA = smem + s * kStageBytes;
      uint8_t* sB = sA + kABytes;
      tc::mbar_expect_tx(full_bar + s, kABytes + b_bytes);
      if (A_MN) {
        tc::tma_load_2d(sA, &tmA, full_bar + s, m0, kb * kBK);
        tc::tma_load_2d(sA + 8192, &tmA, full_bar + s, m0 + 64, kb * kBK);
      } else {
        tc::tma_load_2d(sA, &tmA, full_bar + s, kb * kBK, m0);
      }
      if (B_MN) {
        for (int i = 0; i < p.BN / 64; ++i) tc::tma_load_2d(sB + i * 8192, &tmB, full_bar + s, n0 + 64 * i, kb * kBK);
      } else {
        tc::tma_load_2d(sB, &tmB, full_bar + s, kb * kBK, n0);
      }
    }
  } else if (warp == 1 && lane == 0 && has_work) {
    // ---------------- MMA issuer
    const uint32_t idesc = tc::make_idesc(0, A_MN ? 1 : 0, B_MN ? 1 : 0, kBM, p.BN);
    for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
      const int s = it % kStages;
      const uint32_t ph = (it / kStages) & 1;
      if (!tc::mbar_wait(full_bar + s, ph, aborted, p.status, tc::SITE_FULL, kb)) break;
      tc::tc_fence_after();
      const uint32_t sA = tc::smem_u32(smem + s * kStageBytes);
      const uint32_t sB = sA + kABytes;
#pragma unroll
      for (int k = 0; k < kBK / 16; ++k) {
        const uint64_t ad = A_MN ? tc::make_smem_desc(sA + k * 2048, 8192, 1024) : tc::make_smem_desc(sA + k * 32, 16, 1024);
        const uint64_t bd = B_MN ? tc::make_smem_desc(sB + k * 2048, 8192, 1024) : tc::make_smem_desc(sB + k * 32, 16, 1024);
        tc::umma_f16(tmem_base, ad, bd, idesc, (it > 0 || k > 0) ? 1u : 0u);
      }
      tc::umma_commit(empty_bar + s);   // frees the smem stage once these MMAs have read it
    }
    if (!aborted) tc::umma_commit(tmem_full_bar);
  } else if (warp >= 2 && has_work) {
    // ---------------- epilogue: TMEM -> registers -> fused math -> global
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may read
    const int r = quarter * 32 + lane;            // row of the 128-row tile
    const int row = m0 + r;
    const bool ok = tc::mbar_wait(tmem_full_bar, 0, aborted, p.status, tc::SITE_TMEM_FULL, 0);
    tc::tc_fence_after();
    if (ok) {
      const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16);
      float loss = 0.f;
      float lr = 0.f, scale = 1.f;
      if (MODE == MODE_DW) lr = p.hp[HP_LR_XFC];
      if (MODE == MODE_DX) scale = p.hp[HP_SCALE];
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        float v[32];
        tc::tmem_ld32(tbase + c0, v);
        const int col0 = n0 + c0;
        if (MODE == MODE_LOGITS) {
          if (row < p.M) {
            if (p.loss_acc != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) loss += fmaxf(v[j], 0.f) + log1pf(__expf(-fabsf(v[j])));
            }
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              const int c = col0 + 8 * j8;
              if (c < p.ldG) {
                uint4 pk;
                __half2* h2 = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float a = (c + 2 * j < p.N) ? 1.f / (1.f + __expf(-v[8 * j8 + 2 * j])) : 0.f;
                  const float b = (c + 2 * j + 1 < p.N) ? 1.f / (1.f + __expf(-v[8 * j8 + 2 * j + 1])) : 0.f;
                  h2[j] = __floats2half2_rn(a, b);
                }
                *reinterpret_cast<uint4*>(p.Gt + (size_t)row * p.ldG + c) = pk;
              }
            }
          }
        } else if (MODE == MODE_RAW) {
          // batch-major store Zt[b, label]: for a fixed j the 32 lanes write 32 consecutive labels
          if (row < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) p.Zout[(size_t)(col0 + j) * p.ldG + row] = v[j];
          }
        } else if (MODE == MODE_DX) {
          if (row < p.M) {
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const int c = col0 + 4 * j4;
              if (c < p.N)
                red_add_v4(p.dX + (size_t)row * p.ldX + c, v[4 * j4] * scale, v[4 * j4 + 1] * scale,
                           v[4 * j4 + 2] * scale, v[4 * j4 + 3] * scale);
            }
          }
        } else {  // MODE_DW: fused SGD with momentum and L2 weight decay on the fp16 tiles
          if (row < p.M) {
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              const int c = col0 + 8 * j8;
              if (c < p.N) {
                __half* wp = p.W + (size_t)row * p.ldW + c;
                __half* mp = p.Mom + (size_t)row * p.ldW + c;
                uint4 wr = *reinterpret_cast<const uint4*>(wp);
                uint4 mr = *reinterpret_cast<const uint4*>(mp);
                __half2* w2 = reinterpret_cast<__half2*>(&wr);
                __half2* m2 = reinterpret_cast<__half2*>(&mr);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 w = __half22float2(w2[j]);
                  float2 m = __half22float2(m2[j]);
                  const float g0 = v[8 * j8 + 2 * j] + p.wd * w.x;
                  const float g1 = v[8 * j8 + 2 * j + 1] + p.wd * w.y;
                  m.x = p.mo * m.x + g0;
                  m.y = p.mo * m.y + g1;
                  m2[j] = __floats2half2_rn(m.x, m.y);
                  const float2 mr2 = __half22float2(m2[j]);   // the update uses the stored (rounded) momentum
                  w2[j] = __floats2half2_rn(w.x - lr * mr2.x, w.y - lr * mr2.y);
                }
                *reinterpret_cast<uint4*>(wp) = wr;
                *reinterpret_cast<uint4*>(mp) = mr;
              }
            }
          }
        }
      }
      if (MODE == MODE_LOGITS && p.loss_acc != nullptr) {
        loss = warp_sum(loss);
        if (lane == 0) atomicAdd(p.loss_acc, loss);
      }
    }
    if (MODE == MODE_LOGITS) {
      // all four epilogue warps have stored their rows: subtract 1 at this tile's positives
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ok && p.pos_labels != nullptr) {
        const int nnz = *p.nnz_ptr;
        const int lab_lo = p.label0 + m0;
        const int lab_hi = p.label0 + min(m0 + kBM, p.M);
        const int e0 = lower_bound_i32(p.pos_labels, nnz, lab_lo);
        const int e1 = lower_bound_i32(p.pos_labels, nnz, lab_hi);
        for (int e = e0 + (int)threadIdx.x - 64; e < e1; e += 128) {
          const int b = p.pos_rows[e];
          if (b >= n0 && b < min(n0 + p.BN, p.N)) {
            __half* g = p.Gt + (size_t)(p.pos_labels[e] - p.label0) * p.ldG + b;
            *g = __float2half_rn(__half2float(*g) - 1.f);
          }
        }
      }
    }
  }
  if (MODE == MODE_DX && p.done_counter != nullptr) __threadfence_system();   // this CTA's red.adds are visible
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (MODE == MODE_DX && p.done_counter != nullptr && threadIdx.x == 0) {
    // reduce-scatter epilogue: the last CTA of this rank's dX GEMM tells every rank that the partial
    // sums in this rank's buffer are complete
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(p.done_counter, 1u) == total - 1) {
      *p.done_counter = 0u;
      __threadfence_system();
      const uint32_t v = p.tag.value();
      for (int q = 0; q < p.n_peers; ++q)
        st_release_sys(reinterpret_cast<uint32_t*>(p.peer_flags.p[q]) + p.flag_index, v);
    }
  }
}

// ------------------------------------------------------------------------------------ persistent logits GEMM
// Same math as xfc_gemm_kernel<MODE_LOGITS / MODE_RAW> for label chunks of many tiles: one CTA per SM walks the
// tiles tile = blockIdx.x, blockIdx.x + gridDim.x, ...; the shared-memory ring keeps streaming across tile
// boundaries, and TMEM holds TWO accumulators (2 x 256 columns) so that the epilogue of tile i (sigmoid, fp16
// stores, positives) runs under the loads and MMAs of tile i + 1 instead of after them.  Barriers: full / empty per
// ring stage as before, tmem_full[2] (MMA warp -> epilogue, one commit) and tmem_empty[2] (epilogue -> MMA warp,
// one arrival per epilogue warp).  Opt-in (rb_xfc_set_persistent), off by default.
constexpr int kAccBufs = 2;
constexpr int kTmemColsPersistent = kAccBufs * 256;

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
xfc_logits_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                             const GemmParams p, const int n_m_tiles, const int n_n_tiles) {
  static_assert(MODE == MODE_LOGITS || MODE == MODE_RAW, "logits modes only");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;       // [kAccBufs]
  uint64_t* tmem_empty_bar = tmem_full_bar + kAccBufs; // [kAccBufs]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_empty_bar + kAccBufs);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = n_m_tiles * n_n_tiles;
  const uint32_t b_bytes = (uint32_t)p.BN * kBK * 2;

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
    for (int s = 0; s < kStages; ++s) { tc::mbar_init(full_bar + s, 1); tc::mbar_init(empty_bar + s, 1); }
    for (int a = 0; a < kAccBufs; ++a) { tc::mbar_init(tmem_full_bar + a, 1); tc::mbar_init(tmem_empty_bar + a, 4); }
    *s_abort = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_ptr_smem, kTmemColsPersistent);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  bool aborted = false;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer: one continuous stream of (tile, k block) stages
    if (MODE == MODE_LOGITS && p.wait_flags != nullptr) {
      const uint32_t want = p.tag.value();
      for (int q = 0; q < p.wait_n; ++q)
        if (!wait_flag(p.wait_flags + q, want, p.status, 100 + q)) aborted = true;
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles && !aborted; tile += gridDim.x) {
      const int m0 = (tile / n_n_tiles) * kBM, n0 = (tile % n_n_tiles) * p.BN;
      for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!tc::mbar_wait(empty_bar + s, ph ^ 1, aborted, p.status, tc::SITE_EMPTY, kb)) break;
        uint8_t* sA = smem + s * kStageBytes;
        uint8_t* sB = sA + kABytes;
        tc::mbar_expect_tx(full_bar + s, kABytes + b_bytes);
        tc::tma_load_2d(sA, &tmA, full_bar + s, kb * kBK, m0);
        tc::tma_load_2d(sB, &tmB, full_bar + s, kb * kBK, n0);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer: accumulator t_local & 1, reused every second tile once the epilogue has drained it
    const uint32_t idesc = tc::make_idesc(0, 0, 0, kBM, p.BN);
    int it = 0, t_local = 0;
    for (int tile = blockIdx.x; tile < n_tiles && !aborted; tile += gridDim.x, ++t_local) {
      const int buf = t_local & 1;
      const uint32_t use = (uint32_t)(t_local >> 1);
      if (!tc::mbar_wait(tmem_empty_bar + buf, (use & 1) ^ 1, aborted, p.status, tc::SITE_TMEM_EMPTY, tile)) break;
      tc::tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)buf * 256u;
      for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!tc::mbar_wait(full_bar + s, ph, aborted, p.status, tc::SITE_FULL, kb)) break;
        tc::tc_fence_after();
        const uint32_t sA = tc::smem_u32(smem + s * kStageBytes);
        const uint32_t sB = sA + kABytes;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          const uint64_t ad = tc::make_smem_desc(sA + k * 32, 16, 1024);
          const uint64_t bd = tc::make_smem_desc(sB + k * 32, 16, 1024);
          tc::umma_f16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        tc::umma_commit(empty_bar + s);
      }
      if (aborted) break;
      tc::umma_commit(tmem_full_bar + buf);
    }
  } else if (warp >= 2) {
    // ---------------- epilogue warps: TMEM lane quarter each; all four take the same decisions (named barrier 1)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    float loss = 0.f;
    int t_local = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t_local) {
      const int m0 = (tile / n_n_tiles) * kBM, n0 = (tile % n_n_tiles) * p.BN;
      const int row = m0 + r;
      const int buf = t_local & 1;
      const uint32_t use = (uint32_t)(t_local >> 1);
      if (!tc::mbar_wait(tmem_full_bar + buf, use & 1, aborted, p.status, tc::SITE_TMEM_FULL, tile)) *s_abort = 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*s_abort) break;                                  // the same answer in all four warps
      tc::tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * 256u;
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        float v[32];
        tc::tmem_ld32(tbase + c0, v);
        const int col0 = n0 + c0;
        if (MODE == MODE_LOGITS) {
          if (row < p.M) {
            if (p.loss_acc != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) loss += fmaxf(v[j], 0.f) + log1pf(__expf(-fabsf(v[j])));
            }
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              const int c = col0 + 8 * j8;
              if (c < p.ldG) {
                uint4 pk;
                __half2* h2 = reinterpret_cast<__half2*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float a = (c + 2 * j < p.N) ? 1.f / (1.f + __expf(-v[8 * j8 + 2 * j])) : 0.f;
                  const float b = (c + 2 * j + 1 < p.N) ? 1.f / (1.f + __expf(-v[8 * j8 + 2 * j + 1])) : 0.f;
                  h2[j] = __floats2half2_rn(a, b);
                }
                *reinterpret_cast<uint4*>(p.Gt + (size_t)row * p.ldG + c) = pk;
              }
            }
          }
        } else {
          if (row < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) p.Zout[(size_t)(col0 + j) * p.ldG + row] = v[j];
          }
        }
      }
      // every tcgen05.ld of this tile has completed (tmem_ld32 waits): hand the accumulator back to the MMA warp
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(tmem_empty_bar + buf);
      if (MODE == MODE_LOGITS) {
        asm volatile("bar.sync 1, 128;" ::: "memory");      // all four warps have stored their rows of this tile
        if (p.pos_labels != nullptr) {
          const int nnz = *p.nnz_ptr;
          const int lab_lo = p.label0 + m0;
          const int lab_hi = p.label0 + min(m0 + kBM, p.M);
          const int e0 = lower_bound_i32(p.pos_labels, nnz, lab_lo);
          const int e1 = lower_bound_i32(p.pos_labels, nnz, lab_hi);
          for (int e = e0 + (int)threadIdx.x - 64; e < e1; e += 128) {
            const int b = p.pos_rows[e];
            if (b >= n0 && b < min(n0 + p.BN, p.N)) {
              __half* g = p.Gt + (size_t)(p.pos_labels[e] - p.label0) * p.ldG + b;
              *g = __float2half_rn(__half2float(*g) - 1.f);
            }
          }
        }
      }
    }
    if (MODE == MODE_LOGITS && p.loss_acc != nullptr) {
      loss = warp_sum(loss);
      if (lane == 0) atomicAdd(p.loss_acc, loss);
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, kTmemColsPersistent);
  }
}

// ------------------------------------------------------------------------------------ dW + SGD, W/M tiles staged by TMA
// Same math as xfc_gemm_kernel<MODE_DW>, restructured because the kernel is bound by the W / momentum
// traffic, not by the MMA: the producer warp first issues TMA loads of this CTA's [128 x <=256] tiles of W
// and M into shared memory (they arrive while the short K loop over the batch runs), the epilogue updates
// them in place from the TMEM accumulator (16-byte accesses on the 128-byte-swizzled panels, conflict
// free), and one thread writes both tiles back with TMA stores.  Every global access is a full-line
// bulk copy instead of 16-byte pieces at a 1.5 KB stride.
constexpr int kPanelBytes = kBM * 64 * 2;                        // 128 rows x 64 fp16 = 16 KB
// BN_T = widest N tile the instantiation can hold (128: two CTAs per SM, so one CTA's loads/stores overlap
// the other's epilogue; 256: one CTA per SM), STAGES = depth of the operand ring of the short K loop.
template <int BN_T, int STAGES> struct DwCfg {
  static constexpr int kStage = kABytes + BN_T * kBK * 2;
  static constexpr int kTile = (BN_T / 64) * kPanelBytes;
  static constexpr int kSmem = STAGES * kStage + 2 * kTile + 1024 + 128;
  static constexpr int kTmem = BN_T;
};

template <int BN_T, int STAGES>
__global__ void __launch_bounds__(kThreads, (BN_T <= 128 ? 2 : 1))
xfc_dw_sgd_tma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmM,
                      const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using C = DwCfg<BN_T, STAGES>;
  constexpr int kDwStages = STAGES;
  constexpr int kDwStage = C::kStage;
  uint8_t* sW = smem + kDwStages * kDwStage;
  uint8_t* sM = sW + C::kTile;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sM + C::kTile);
  uint64_t* empty_bar = full_bar + kDwStages;
  uint64_t* tmem_full_bar = empty_bar + kDwStages;
  uint64_t* wm_full_bar = tmem_full_bar + 1;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(wm_full_bar + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kBM;
  const int n0 = blockIdx.y * p.BN;
  const int panels = p.BN / 64;
  const uint32_t b_bytes = (uint32_t)p.BN * kBK * 2;

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmA); tc::prefetch_tmap(&tmB); tc::prefetch_tmap(&tmW); tc::prefetch_tmap(&tmM);
    for (int s = 0; s < kDwStages; ++s) { tc::mbar_init(full_bar + s, 1); tc::mbar_init(empty_bar + s, 1); }
    tc::mbar_init(tmem_full_bar, 1);
    tc::mbar_init(wm_full_bar, 1);
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_ptr_smem, C::kTmem);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  bool aborted = false;

  if (warp == 0 && lane == 0) {
    tc::mbar_expect_tx(wm_full_bar, (uint32_t)panels * 2 * kPanelBytes);
    for (int q = 0; q < panels; ++q) {
      tc::tma_load_2d(sW + q * kPanelBytes, &tmW, wm_full_bar, n0 + 64 * q, m0);
      tc::tma_load_2d(sM + q * kPanelBytes, &tmM, wm_full_bar, n0 + 64 * q, m0);
    }
    for (int kb = 0; kb < p.kb_total; ++kb) {
      const int s = kb % kDwStages;
      const uint32_t ph = (kb / kDwStages) & 1;
      if (!tc::mbar_wait(empty_bar + s, ph ^ 1, aborted, p.status, tc::SITE_EMPTY, kb)) break;
      uint8_t* sA = smem + s * kDwStage;
      uint8_t* sB = sA + kABytes;
      tc::mbar_expect_tx(full_bar + s, kABytes + b_bytes);
      tc::tma_load_2d(sA, &tmA, full_bar + s, kb * kBK, m0);
      for (int i = 0; i < panels; ++i) tc::tma_load_2d(sB + i * 8192, &tmB, full_bar + s, n0 + 64 * i, kb * kBK);
    }
  } else if (warp == 1 && lane == 0) {
    const uint32_t idesc = tc::make_idesc(0, 0, 1, kBM, p.BN);
    for (int kb = 0; kb < p.kb_total; ++kb) {
      const int s = kb % kDwStages;
      const uint32_t ph = (kb / kDwStages) & 1;
      if (!tc::mbar_wait(full_bar + s, ph, aborted, p.status, tc::SITE_FULL, kb)) break;
      tc::tc_fence_after();
      const uint32_t sA = tc::smem_u32(smem + s * kDwStage);
      const uint32_t sB = sA + kABytes;
#pragma unroll
      for (int k = 0; k < kBK / 16; ++k) {
        const uint64_t ad = tc::make_smem_desc(sA + k * 32, 16, 1024);
        const uint64_t bd = tc::make_smem_desc(sB + k * 2048, 8192, 1024);
        tc::umma_f16(tmem_base, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
      }
      tc::umma_commit(empty_bar + s);
    }
    if (!aborted) tc::umma_commit(tmem_full_bar);
  } else if (warp >= 2) {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    bool ok = tc::mbar_wait(tmem_full_bar, 0, aborted, p.status, tc::SITE_TMEM_FULL, 0);
    ok = tc::mbar_wait(wm_full_bar, 0, aborted, p.status, tc::SITE_FULL, 1000) && ok;
    tc::tc_fence_after();
    if (ok) {
      const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const float lr = p.hp[HP_LR_XFC];
      const uint32_t sr_seed = reinterpret_cast<const uint32_t*>(p.hp)[HP_SEED];
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        float v[32];
        tc::tmem_ld32(tbase + c0, v);
        const int panel = c0 >> 6;
        const int chunk0 = (c0 & 63) >> 3;            // first 16-byte chunk of this 32-column group in the panel row
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const int phys = (chunk0 + j8) ^ (r & 7);   // 128-byte swizzle: chunk index XOR row-in-group
          const uint32_t off = (uint32_t)panel * kPanelBytes + (uint32_t)r * 128 + (uint32_t)phys * 16;
          uint4 wr = *reinterpret_cast<const uint4*>(sW + off);
          uint4 mr = *reinterpret_cast<const uint4*>(sM + off);
          __half2* w2 = reinterpret_cast<__half2*>(&wr);
          __half2* m2 = reinterpret_cast<__half2*>(&mr);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 w = __half22float2(w2[j]);
            float2 m = __half22float2(m2[j]);
            const float g0 = v[8 * j8 + 2 * j] + p.wd * w.x;
            const float g1 = v[8 * j8 + 2 * j + 1] + p.wd * w.y;
            m.x = p.mo * m.x + g0;
            m.y = p.mo * m.y + g1;
            m2[j] = __floats2half2_rn(m.x, m.y);
            const float2 ms = __half22float2(m2[j]);
            if (p.stochastic_round) {
              const uint32_t e = (uint32_t)(m0 + r) * (uint32_t)p.ldW + (uint32_t)(n0 + c0 + 8 * j8 + 2 * j);
              w2[j] = __halves2half2(sr_half(w.x - lr * ms.x, mix32(sr_seed, 0x5152u, e)),
                                     sr_half(w.y - lr * ms.y, mix32(sr_seed, 0x5152u, e + 1)));
            } else {
              w2[j] = __floats2half2_rn(w.x - lr * ms.x, w.y - lr * ms.y);
            }
          }
          *reinterpret_cast<uint4*>(sW + off) = wr;
          *reinterpret_cast<uint4*>(sM + off) = mr;
        }
      }
      tc::fence_proxy_async();     // the tiles were written through the generic proxy; TMA reads them through the async one
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (ok && threadIdx.x == 64) {
      for (int q = 0; q < panels; ++q) {
        if (n0 + 64 * q < p.N) {
          tc::tma_store_2d(&tmW, sW + q * kPanelBytes, n0 + 64 * q, m0);
          tc::tma_store_2d(&tmM, sM + q * kPanelBytes, n0 + 64 * q, m0);
        }
      }
      tc::tma_store_commit_and_wait_read();
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem_base, C::kTmem);
  }
}

// ------------------------------------------------------------------------------------ row-wise top-k by radix select
// One CTA per batch row scans that row of the batch-major logits chunk (L2 resident) five times: four
// 8-bit histogram passes find the k-th largest key exactly, the fifth collects every element above it
// plus as many ties as needed.  Output is unordered (the cross-chunk / cross-rank merge sorts k items).
// Replaces torch.topk / the K passes of torch.max + index_put_ of the reference (dl_base.py:745-756).
__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(256) topk_rows_kernel(const float* __restrict__ Z, int ldZ, int n, int k, int label0,
                                                        float* __restrict__ out_val, int* __restrict__ out_idx) {
  __shared__ unsigned hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_remaining, s_cnt_gt, s_cnt_eq;
  const float* row = Z + (size_t)blockIdx.x * ldZ;
  float* ov = out_val + (size_t)blockIdx.x * k;
  int* oi = out_idx + (size_t)blockIdx.x * k;
  const int kk = min(k, n);
  if (threadIdx.x == 0) { s_prefix = 0u; s_mask = 0u; s_remaining = kk; s_cnt_gt = 0; s_cnt_eq = 0; }
  for (int i = kk + (int)threadIdx.x; i < k; i += blockDim.x) { ov[i] = -3.0e38f; oi[i] = label0; }
  __syncthreads();
  for (int pass = 3; pass >= 0; --pass) {
    hist[threadIdx.x] = 0u;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = order_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 0xFFu], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int remaining = s_remaining;
      int d = 255;
      for (; d > 0; --d) {
        if ((int)hist[d] >= remaining) break;
        remaining -= (int)hist[d];
      }
      s_remaining = remaining;
      s_prefix = prefix | ((uint32_t)d << (8 * pass));
      s_mask = mask | (0xFFu << (8 * pass));
    }
    __syncthreads();
  }
  const uint32_t T = s_prefix;
  const int need_eq = s_remaining;
  const int n_gt = kk - need_eq;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float x = row[i];
    const uint32_t key = order_key(x);
    if (key > T) {
      const int slot = atomicAdd(&s_cnt_gt, 1);
      if (slot < n_gt) { ov[slot] = x; oi[slot] = label0 + i; }
    } else if (key == T) {
      const int slot = atomicAdd(&s_cnt_eq, 1);
      if (slot < need_eq) { ov[n_gt + slot] = x; oi[n_gt + slot] = label0 + i; }
    }
  }
}

// sum over positives of z = W[label] . X[row]  (only on loss-sampling steps): one warp per positive
__global__ void xfc_pos_logit_sum_kernel(const __half* __restrict__ W, const __half* __restrict__ X, int D,
                                         const int* __restrict__ pos_rows, const int* __restrict__ pos_labels,
                                         const int* __restrict__ nnz_ptr, float* __restrict__ loss_acc) {
  const int nnz = *nnz_ptr;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  float total = 0.f;
  for (int e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; e < nnz; e += warps) {
    const __half* w = W + (size_t)pos_labels[e] * D;
    const __half* x = X + (size_t)pos_rows[e] * D;
    float a = 0.f;
    for (int d = lane * 2; d < D; d += 64) {
      const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(w + d));
      const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(x + d));
      a += wf.x * xf.x + wf.y * xf.y;
    }
    total += warp_sum(a);
  }
  if (lane == 0 && total != 0.f) atomicAdd(loss_acc, -total);
}

}  // namespace rb

using namespace rb;

template <int MODE>
static int launch_gemm(const CUtensorMap& a, const CUtensorMap& b, const GemmParams& p, dim3 grid, cudaStream_t st) {
  static bool attr_set = false;
  auto k = xfc_gemm_kernel<MODE>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return -5;
    attr_set = true;
  }
  k<<<grid, kThreads, kSmemBytes, st>>>(a, b, p);
  return 0;
}

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

static int g_xfc_persistent = 0;
// Chooses the persistent logits kernel for chunks with more tiles than SMs (0 = off, the default).
RB_API void rb_xfc_set_persistent(int on) { g_xfc_persistent = on ? 1 : 0; }
RB_API int rb_xfc_get_persistent(void) { return g_xfc_persistent; }

template <int MODE>
static int launch_persistent(const CUtensorMap& a, const CUtensorMap& b, const GemmParams& p, int n_m_tiles, int n_n_tiles,
                             cudaStream_t st) {
  static bool attr_set = false;
  auto k = xfc_logits_persistent_kernel<MODE>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return -5;
    attr_set = true;
  }
  const int n_tiles = n_m_tiles * n_n_tiles;
  const int ctas = n_tiles < sm_count() ? n_tiles : sm_count();
  k<<<ctas, kThreads, kSmemBytes, st>>>(a, b, p, n_m_tiles, n_n_tiles);
  return 0;
}

// Gt[Lc, ldG] = sigmoid(W X^T) - Y for the label chunk W[Lc, D]; labels of the chunk are
// label0 .. label0+Lc-1 in the numbering of pos_labels.  raw_out != null writes fp32 logits instead
// (no sigmoid, no positives), batch-major, into raw_out[B, ldG] with ldG >= Lc.
RB_API int rb_xfc_logits_grad(const void* W, int Lc, int D, const void* X, int B, void* Gt, int ldG,
                              const int* pos_rows, const int* pos_labels, const int* nnz_ptr, int label0,
                              float* loss_acc, float* raw_out, const unsigned* wait_flags, int wait_n,
                              const unsigned* step_ptr, int* status, cudaStream_t st) {
  if (D % 8 || ldG % 8 || Lc < 1 || B < 1) return -3;
  if (raw_out == nullptr ? ldG < B : ldG < Lc) return -3;
  const int BN = B >= 256 ? 256 : round_up(B, 16);
  CUtensorMap ta, tb;
  int rc = tc::make_tmap_2d(&ta, W, Lc, D, D, 64, kBM, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&tb, X, B, D, D, 64, BN, false);
  if (rc) return rc;
  GemmParams p{};
  p.M = Lc; p.N = B; p.BN = BN; p.kb_total = (D + kBK - 1) / kBK; p.kb_per_split = p.kb_total; p.status = status;
  p.Gt = (__half*)Gt; p.ldG = ldG; p.pos_rows = pos_rows; p.pos_labels = pos_labels; p.nnz_ptr = nnz_ptr;
  p.label0 = label0; p.loss_acc = loss_acc; p.Zout = raw_out;
  p.wait_flags = wait_flags; p.wait_n = wait_n; p.tag = StepTag{step_ptr, 1u, 0u};
  dim3 grid((Lc + kBM - 1) / kBM, (B + BN - 1) / BN, 1);
  if (g_xfc_persistent && (int)(grid.x * grid.y) > sm_count()) {
    // more tiles than SMs: one persistent CTA per SM, epilogues overlapped with the next tile's main loop
    rc = raw_out ? launch_persistent<MODE_RAW>(ta, tb, p, (int)grid.x, (int)grid.y, st)
                 : launch_persistent<MODE_LOGITS>(ta, tb, p, (int)grid.x, (int)grid.y, st);
  } else {
    rc = raw_out ? launch_gemm<MODE_RAW>(ta, tb, p, grid, st) : launch_gemm<MODE_LOGITS>(ta, tb, p, grid, st);
  }
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_xfc_pos_logit_sum(const void* W, const void* X, int D, const int* pos_rows, const int* pos_labels,
                                const int* nnz_ptr, float* loss_acc, cudaStream_t st) {
  if (D % 2) return -3;
  xfc_pos_logit_sum_kernel<<<64, 128, 0, st>>>((const __half*)W, (const __half*)X, D, pos_rows, pos_labels, nnz_ptr,
                                               loss_acc);
  RB_LAUNCH_CHECK();
  return 0;
}

// dX[B, D] += hp[SCALE] * Gt^T W over the chunk (dX must have been zeroed before the first chunk)
// With done_counter != null the last CTA stores the step tag into word flag_index of every peer's flag
// array (the fused reduce-scatter signal; pass it on the final label chunk only).
RB_API int rb_xfc_dx(const void* Gt, int ldG, const void* W, int Lc, int D, int B, float* dX, const float* hp,
                     int splits, unsigned* done_counter, void* const* peer_flags, int n_peers, int flag_index,
                     const unsigned* step_ptr, int* status, cudaStream_t st) {
  if (D % 8 || ldG % 8 || Lc < 1) return -3;
  const int BN = D >= 256 ? 256 : round_up(D, 64);
  CUtensorMap ta, tb;
  int rc = tc::make_tmap_2d(&ta, Gt, Lc, ldG, ldG, 64, 64, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&tb, W, Lc, D, D, 64, 64, false);
  if (rc) return rc;
  GemmParams p{};
  p.M = B; p.N = D; p.BN = BN; p.kb_total = (Lc + kBK - 1) / kBK; p.status = status;
  if (splits < 1) splits = 1;
  if (splits > p.kb_total) splits = p.kb_total;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
  p.dX = dX; p.ldX = D; p.hp = hp;
  if (done_counter != nullptr) {
    if (n_peers > kMaxPeers) return -3;
    p.done_counter = done_counter; p.n_peers = n_peers; p.flag_index = flag_index; p.tag = StepTag{step_ptr, 1u, 0u};
    for (int q = 0; q < n_peers; ++q) p.peer_flags.p[q] = peer_flags[q];
  }
  dim3 grid((B + kBM - 1) / kBM, (D + BN - 1) / BN, splits);
  rc = launch_gemm<MODE_DX>(ta, tb, p, grid, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// W, Mom [Lc, D] updated in place from dW = Gt X (never stored); lr read from hp[LR_XFC]
// use_tma_tiles: 0 = epilogue reads/writes W and M directly; 1 = TMA-staged 128-column tiles, two CTAs per SM
// (default); 2 = TMA-staged 256-column tiles, one CTA per SM.
RB_API int rb_xfc_dw_sgd(const void* Gt, int ldG, const void* X, int B, void* W, void* Mom, int Lc, int D,
                         const float* hp, float mo, float wd, int use_tma_tiles, int stochastic_round, int* status,
                         cudaStream_t st) {
  if (D % 8 || ldG % 8 || Lc < 1) return -3;
  const int bn_max = (use_tma_tiles == 1) ? 128 : 256;
  const int BN = D >= bn_max ? bn_max : round_up(D, 64);
  CUtensorMap ta, tb;
  int rc = tc::make_tmap_2d(&ta, Gt, Lc, ldG, ldG, 64, kBM, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&tb, X, B, D, D, 64, 64, false);
  if (rc) return rc;
  GemmParams p{};
  p.M = Lc; p.N = D; p.BN = BN; p.kb_total = (B + kBK - 1) / kBK; p.kb_per_split = p.kb_total; p.status = status;
  p.W = (__half*)W; p.Mom = (__half*)Mom; p.ldW = D; p.hp = hp; p.mo = mo; p.wd = wd;
  p.stochastic_round = stochastic_round;
  if (stochastic_round && !use_tma_tiles) return -3;
  dim3 grid((Lc + kBM - 1) / kBM, (D + BN - 1) / BN, 1);
  if (use_tma_tiles) {
    CUtensorMap tw, tm;
    rc = tc::make_tmap_2d(&tw, W, Lc, D, D, 64, kBM, false);
    if (rc) return rc;
    rc = tc::make_tmap_2d(&tm, Mom, Lc, D, D, 64, kBM, false);
    if (rc) return rc;
    if (use_tma_tiles == 2) {
      using C = DwCfg<256, 2>;
      static bool attr_set = false;
      if (!attr_set) {
        if (cudaFuncSetAttribute(xfc_dw_sgd_tma_kernel<256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
          return -5;
        attr_set = true;
      }
      xfc_dw_sgd_tma_kernel<256, 2><<<grid, kThreads, C::kSmem, st>>>(ta, tb, tw, tm, p);
    } else {
      using C = DwCfg<128, 1>;
      static bool attr_set = false;
      if (!attr_set) {
        if (cudaFuncSetAttribute(xfc_dw_sgd_tma_kernel<128, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem) != cudaSuccess)
          return -5;
        attr_set = true;
      }
      xfc_dw_sgd_tma_kernel<128, 1><<<grid, kThreads, C::kSmem, st>>>(ta, tb, tw, tm, p);
    }
  } else {
    rc = launch_gemm<MODE_DW>(ta, tb, p, grid, st);
    if (rc) return rc;
  }
  RB_LAUNCH_CHECK();
  return 0;
}

// Unordered top-k of every row of the batch-major fp32 logits Z[B, ldZ] (first n columns valid).
RB_API int rb_topk_rows(const float* Z, int ldZ, int B, int n, int k, int label0, float* out_val, int* out_idx,
                        cudaStream_t st) {
  if (B < 1 || n < 1 || k < 1) return -3;
  topk_rows_kernel<<<B, 256, 0, st>>>(Z, ldZ, n, k, label0, out_val, out_idx);
  RB_LAUNCH_CHECK();
  return 0;
}
