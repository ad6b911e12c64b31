// GEMMs for sm_100a: one persistent tcgen05 / TMEM kernel family with the element-wise neighbours of every linear
// layer of the encoder, and the three products of the classifier step, fused into the epilogue.  They stand in for the cuBLAS calls behind the reference's HF
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
//              GELU_BWD             C = acc * gelu'(R) ;  column sums of C -> bias gradient accumulators
//              SPLITK               fp32 partials reduced in L2, the last CTA of a tile converts and stores
//              SIGMOID_POS          C = sigmoid(acc) - Y: the classifier's logit gradient; Y from a label-sorted list of
//                                   positives applied to the staged tile in shared memory before it is stored; on
//                                   loss-sampling steps also the sum of softplus(acc) (parity: dl_base.py:572-594)
//              DX                   dX += scale * acc by vector reductions into an fp32 matrix (contraction over the
//                                   labels of a chunk, split over the CTAs); the last CTA raises the peers' flags
//              DW_SGD               classifier weights: W and momentum tiles [128 x 64] come in by TMA under the main loop,
//                                   m = mo m + (acc + wd w), w -= lr m (stochastic rounding optional) in shared memory,
//                                   both tiles leave by TMA; dW = Gt X is never stored (parity: dl_base.py:623-633, 343-344)
//              TOPK                 nothing is stored: every epilogue thread keeps the 8 largest entries of its row
//                                   over all the tiles its CTA visits and writes them as candidates at the end
//                                   (prediction: X W^T is never materialised; parity: dl_base.py:745-756)
//
// Structure.  Persistent CTAs walk the work items (tile x K-split).  576 threads: warp 0 TMA producer, warp 1
// TMEM owner + MMA issuer, warps 2..17 epilogue (four groups of four warps, one TMEM lane quarter per warp, one
// 64-column panel of the tile per group: the epilogue is bound by instruction latency, not by issue slots, and
// sixteen warps hide what eight could not).  The shared-memory ring keeps streaming across item boundaries and TMEM
// holds two accumulators, so the epilogue of item i runs under the main loop of item i + 1.
//
// Two tile shapes.  NCTA = 1: a CTA owns a 128 x BN tile.  NCTA = 2 (`cta_group::2`): the two CTAs of a cluster
// of two own a 256 x BN tile; each loads its 128 rows of A and HALF of the B columns, the leader CTA issues
// MMAs that read both CTAs' shared memory and write 128 accumulator rows into each CTA's TMEM.  The kernel is
// bound by the rate at which an SM can fetch operand rows, and the pair fetches 128 + BN/2 rows per k block and
// CTA instead of 128 + BN for the same MMA work.  Loads are plain TMA tile loads (no multicast); a pair's loads
// count their bytes on the leader's barrier and one `tcgen05.commit` arrives on both CTAs' barriers.
//
// Epilogue.  Output tiles are staged in 128-byte-swizzled shared-memory panels ([128 rows x 64 columns] of 16-bit
// elements) and written with TMA stores, which clip at the matrix edge; tile-shaped inputs (residual, stored
// pre-activation) are fetched into the same panels by TMA while the tile's main loop still runs and are updated
// in place.  Every global access of the epilogue is therefore a full-line bulk copy.
//
// Every wait is bounded (tc.cuh): a protocol error ends with a status word, never with a hang.
#include <type_traits>
#include "peer.cuh"

namespace rb {
namespace eg {

constexpr int BM = 128;                         // accumulator rows per CTA
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;            // 16 KB
constexpr int PANEL_BYTES = BM * 64 * 2;        // one staging panel: 128 rows x 64 x 16 bit
constexpr int EGROUPS = 4;                      // epilogue groups of four warps (one per TMEM lane quarter)
constexpr int N_PANELS = EGROUPS;               // one staging panel per epilogue group
constexpr int EPI_THREADS = 128 * EGROUPS;
constexpr int THREADS = 64 + EPI_THREADS;       // producer warp, MMA warp, sixteen epilogue warps
constexpr int ACC_BUFS = 2;
constexpr int ACC_STRIDE = 256;                 // TMEM columns between the two accumulators
constexpr int TMEM_COLS = ACC_BUFS * ACC_STRIDE;

// Shared memory: the operand ring plus, for epilogues that stage tiles, one panel per epilogue group.  The main
// loop is bound by load latency over the bytes in flight, so the ring takes everything else (192 KB).
constexpr int RING_BYTES = 192 * 1024;          // operand bytes in flight per CTA
constexpr int MAX_STAGES = 8;                   // a stage is 16 KB of A + BN / NCTA rows of B: 24 KB (8 stages) .. 48 KB (4)

enum Layout : int { L_NT = 0, L_NN = 1, L_TN = 2 };
enum Epi : int { E_STORE = 0, E_BIAS_GELU = 1, E_BIAS_DROPOUT_RESID = 2, E_ADD = 3, E_GELU_BWD = 4, E_SPLITK = 5, E_TOPK = 6, E_SIGMOID_POS = 7, E_DX = 8, E_DW_SGD = 9 };

// DW_SGD updates two tile-shaped tensors in place (weights and momentum): two panels per group, a 160 KB ring.
constexpr int SMEM_BUDGET = 224 * 1024;         // ring + panels
constexpr bool staged_epi(int epi) { return epi != E_SPLITK && epi != E_TOPK && epi != E_DX; }
constexpr int panel_count(int epi) { return !staged_epi(epi) ? 0 : (epi == E_DW_SGD ? 2 * N_PANELS : N_PANELS); }
constexpr int ring_bytes(int epi) {
  return SMEM_BUDGET - panel_count(epi) * PANEL_BYTES < RING_BYTES ? SMEM_BUDGET - panel_count(epi) * PANEL_BYTES : RING_BYTES;
}
template <int EPI> struct Cfg {
  static constexpr bool kStaged = staged_epi(EPI);
  static constexpr int kPanels = panel_count(EPI);
  static constexpr int kRing = ring_bytes(EPI);
  static constexpr int kSmem = kRing + kPanels * PANEL_BYTES + 1024 + 512;
};

struct Params {
  int M, N;                      // output rows / columns
  int BN;                        // N tile: 64, 128 or 256 (NCTA = 2: 128 or 256)
  int n_m_tiles, n_n_tiles;      // tiles of (128 NCTA) x BN
  int splits, kb_total, kb_per_split;
  void* C; int ldc;              // direct stores of the split-K fix-up only
  const void* bias;              // [N]                             BIAS_GELU, BIAS_DROPOUT_RESID
  float p; const int* seed; uint32_t stream;        // dropout      BIAS_DROPOUT_RESID
  float* colacc; int col_tot; int col_off;          // GELU_BWD: replicas of [col_tot] floats, this vector at col_off
  float* sk_scratch; unsigned* sk_counters;         // SPLITK: [tiles][128 NCTA x BN] fp32 (zero between launches), [tiles]
  float* cand_val; int* cand_idx; int cand_ld;      // TOPK: [M, cand_ld] candidates, 8 per (CTA, epilogue group)
  // SIGMOID_POS (classifier logits + gradient): label-sorted positives, label id of row 0, all-gather flags to wait for
  const int* pos_rows; const int* pos_labels; const int* nnz_ptr; int label0;
  const uint32_t* wait_flags; int wait_n; const uint32_t* step_ptr;
  float* loss_acc;               // SIGMOID_POS, loss-sampling steps: += sum of softplus(z) over the valid logits
  // DX (classifier input gradient): fp32 accumulation target, loss scale, completion signal to the peers
  float* dX; int ldX; const float* hp;
  unsigned* done_counter; void* peer_flags[16]; int n_peers; int flag_index;
  // DW_SGD (classifier weights): momentum, weight decay, rounding mode; the row stride numbers the elements for the
  // rounding hash; the learning rate and the seed come from hp
  float mo, wd; int stochastic_round; int ldW;
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
template <typename T> __device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
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

// Byte offset of the 16-byte chunk `chunk` (8 columns) of row r inside a 128-byte-swizzled panel.
__device__ __forceinline__ uint32_t panel_off(int r, int chunk) { return (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4); }

template <typename T, int LAYOUT, int EPI, int NCTA>
__global__ void __launch_bounds__(THREADS, 1)
enc_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
                const __grid_constant__ CUtensorMap tmF, const Params p) {
  using C_ = Cfg<EPI>;
  constexpr int RING = C_::kRing;
  constexpr bool A_MN = (LAYOUT == L_TN);
  constexpr bool B_MN = (LAYOUT != L_NT);
  constexpr int FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  constexpr bool HAS_IN = (EPI == E_BIAS_DROPOUT_RESID || EPI == E_ADD || EPI == E_GELU_BWD || EPI == E_DW_SGD);   // tile-shaped input R
  constexpr bool STAGED = C_::kStaged;                                                           // outputs through panels
  constexpr uint32_t IN_BYTES = EPI == E_DW_SGD ? 2 * PANEL_BYTES : PANEL_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* panels = smem + RING;                           // [N_PANELS][PANEL_BYTES], 1024-byte aligned
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(panels + C_::kPanels * PANEL_BYTES);
  uint64_t* empty_bar = full_bar + MAX_STAGES;
  uint64_t* tmem_full_bar = empty_bar + MAX_STAGES;      // [ACC_BUFS]
  uint64_t* tmem_empty_bar = tmem_full_bar + ACC_BUFS;   // [ACC_BUFS]  (used in the leader CTA)
  uint64_t* in_bar = tmem_empty_bar + ACC_BUFS;          // [N_PANELS]  a group's R panel has landed
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(in_bar + N_PANELS);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* s_last = s_abort + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = NCTA == 2 ? tc::cluster_ctarank() : 0u;
  const int unit = NCTA == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;          // which persistent worker
  const int n_units = NCTA == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int n_items = p.n_m_tiles * p.n_n_tiles * p.splits;
  const int b_rows = p.BN / NCTA;                                                 // B rows (N index) this CTA loads
  const int STAGE = A_BYTES + b_rows * BK * 2;                                    // 24, 32 or 48 KB
  const int STAGES = min(MAX_STAGES, RING / STAGE);
  const uint32_t stage_tx = (uint32_t)NCTA * (uint32_t)STAGE;

  if (threadIdx.x == 0) {
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
    if (STAGED) tc::prefetch_tmap(&tmC);
    if (HAS_IN) tc::prefetch_tmap(&tmR);
    if (EPI == E_BIAS_GELU || EPI == E_DW_SGD) tc::prefetch_tmap(&tmF);
    for (int s = 0; s < MAX_STAGES; ++s) { tc::mbar_init(full_bar + s, 1); tc::mbar_init(empty_bar + s, 1); }
    for (int a = 0; a < ACC_BUFS; ++a) { tc::mbar_init(tmem_full_bar + a, 1); tc::mbar_init(tmem_empty_bar + a, 4 * EGROUPS * NCTA); }
    for (int a = 0; a < N_PANELS; ++a) tc::mbar_init(in_bar + a, 1);
    *s_abort = 0;
    *s_last = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    if (NCTA == 2) tc::tmem_alloc_pair(tmem_ptr_smem, TMEM_COLS); else tc::tmem_alloc(tmem_ptr_smem, TMEM_COLS);
  }
  tc::tc_fence_before();
  __syncthreads();
  if (NCTA == 2) tc::cluster_sync_all();            // the peer's barriers exist before anything arrives on them
  tc::tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  bool aborted = false;
  // everything above touched no global memory: it may have run under the tail of the previous kernel
  grid_dep_wait();
  grid_dep_launch();

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer: one continuous stream of (item, k block) stages
    int s = 0;
    uint32_t ph = 0;
    if (EPI == E_SIGMOID_POS && p.wait_flags != nullptr) {
      // all-gather prologue: every rank has pushed its rows of X into this GPU's buffer and raised its flag; the
      // loads below go through the async proxy, hence the proxy fence after the acquire
      const uint32_t want = *p.step_ptr;
      for (int q = 0; q < p.wait_n; ++q)
        if (!wait_flag(p.wait_flags + q, want, p.status, 100 + q)) aborted = true;
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    for (int item = unit; item < n_items && !aborted; item += n_units) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int m0 = (tile / p.n_n_tiles) * (BM * NCTA) + (int)rank * BM;
      const int n0 = (tile % p.n_n_tiles) * p.BN + (int)rank * b_rows;
      const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
        if (!tc::mbar_wait(empty_bar + s, ph ^ 1, aborted, p.status, tc::SITE_EMPTY, kb)) break;
        uint8_t* sA = smem + s * STAGE;
        uint8_t* sB = sA + A_BYTES;
        if (NCTA == 1) {
          tc::mbar_expect_tx(full_bar + s, stage_tx);
          if (A_MN) {
            tc::tma_load_2d(sA, &tmA, full_bar + s, m0, kb * BK);
            tc::tma_load_2d(sA + 8192, &tmA, full_bar + s, m0 + 64, kb * BK);
          } else {
            tc::tma_load_2d(sA, &tmA, full_bar + s, kb * BK, m0);
          }
          if (B_MN) {
            for (int i = 0; i < b_rows / 64; ++i) tc::tma_load_2d(sB + i * 8192, &tmB, full_bar + s, n0 + 64 * i, kb * BK);
          } else {
            tc::tma_load_2d(sB, &tmB, full_bar + s, kb * BK, n0);
          }
        } else {
          // the leader's barrier counts the bytes of both CTAs' loads; only the leader announces them
          const uint32_t lbar = tc::leader_addr(tc::smem_u32(full_bar + s));
          if (rank == 0) tc::mbar_expect_tx(full_bar + s, stage_tx);
          if (A_MN) {
            tc::tma_load_2d_pair(sA, &tmA, lbar, m0, kb * BK);
            tc::tma_load_2d_pair(sA + 8192, &tmA, lbar, m0 + 64, kb * BK);
          } else {
            tc::tma_load_2d_pair(sA, &tmA, lbar, kb * BK, m0);
          }
          if (B_MN) {
            for (int i = 0; i < b_rows / 64; ++i) tc::tma_load_2d_pair(sB + i * 8192, &tmB, lbar, n0 + 64 * i, kb * BK);
          } else {
            tc::tma_load_2d_pair(sB, &tmB, lbar, kb * BK, n0);
          }
        }
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------- MMA issuer (leader CTA): accumulator (t_local & 1), reused once the epilogue(s) drained it
    const uint32_t idesc = tc::make_idesc(FMT, A_MN ? 1 : 0, B_MN ? 1 : 0, BM * NCTA, p.BN);
    int s = 0, t_local = 0;
    uint32_t ph = 0;
    for (int item = unit; item < n_items && !aborted; item += n_units, ++t_local) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int kb0 = split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
      const int buf = t_local & 1;
      const uint32_t use = (uint32_t)(t_local >> 1);
      if (!tc::mbar_wait(tmem_empty_bar + buf, (use & 1) ^ 1, aborted, p.status, tc::SITE_TMEM_EMPTY, item)) break;
      tc::tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)buf * ACC_STRIDE;
      for (int kb = kb0; kb < kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
        if (!tc::mbar_wait(full_bar + s, ph, aborted, p.status, tc::SITE_FULL, kb)) break;
        tc::tc_fence_after();
        const uint32_t sA = tc::smem_u32(smem + s * STAGE);
        const uint32_t sB = sA + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          const uint64_t ad = A_MN ? tc::make_smem_desc(sA + k * 2048, 8192, 1024) : tc::make_smem_desc(sA + k * 32, 16, 1024);
          const uint64_t bd = B_MN ? tc::make_smem_desc(sB + k * 2048, 8192, 1024) : tc::make_smem_desc(sB + k * 32, 16, 1024);
          if (NCTA == 2) tc::umma_f16_pair(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          else tc::umma_f16(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        if (NCTA == 2) tc::umma_commit_pair(empty_bar + s); else tc::umma_commit(empty_bar + s);
      }
      if (aborted) break;
      if (NCTA == 2) tc::umma_commit_pair(tmem_full_bar + buf); else tc::umma_commit(tmem_full_bar + buf);
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: group g = (warp - 2) / 4 owns columns [g BN/2, (g + 1) BN/2) of the CTA's 128 rows
    const int quarter = warp & 3;
    const int g = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;                    // row of the CTA's accumulator = TMEM lane
    // staged epilogues: group g takes the 64-column panel g of the tile (BN / 64 groups have one, the others idle);
    // the others split the tile's columns into BN / EGROUPS (at least 32) per group
    const int n_pan = g < (p.BN >> 6) ? 1 : 0;
    const int g_col = g * 64;
    const int ucols = p.BN / EGROUPS < 32 ? 32 : p.BN / EGROUPS;
    const bool u_active = g * ucols < p.BN;
    const int bar_id = 2 + g;                             // named barrier of this group (128 threads)
    const bool elected = (warp == 2 + 4 * g) && lane == 0;                   // first warp of the group, lane 0
    uint8_t* pan = panels + g * PANEL_BYTES;              // this group's staging panel
    uint8_t* pan2 = panels + (N_PANELS + g) * PANEL_BYTES;   // DW_SGD: the momentum panel beside the weight panel
    uint64_t* my_in_bar = in_bar + g;
    uint32_t seed = 0u;
    float inv_keep = 1.f;
    if (EPI == E_BIAS_DROPOUT_RESID && p.p > 0.f) { seed = (uint32_t)(*p.seed); inv_keep = 1.f / (1.f - p.p); }
    int t_local = 0;
    uint32_t in_count = 0;                                // R panels fetched so far (parity of my_in_bar)
    // TOPK: this thread's 8 best (value, column) of its row so far, sorted descending; cur_m = row block they belong to
    float tv[8];
    int ti[8];
    int cur_m = -1;
    float loss = 0.f;                                     // SIGMOID_POS: this thread's share of sum softplus(z)
    const int slot = ((int)blockIdx.x * EGROUPS + g) * 8;
    for (int item = unit; item < n_items; item += n_units, ++t_local) {
      const int tile = item / p.splits;
      if (EPI == E_TOPK) {
        const int mt = tile / p.n_n_tiles;
        if (mt != cur_m) {
          if (cur_m >= 0) {
            const int frow = cur_m * (BM * NCTA) + (int)rank * BM + r;
            if (frow < p.M && u_active) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                p.cand_val[(size_t)frow * p.cand_ld + slot + k] = tv[k];
                p.cand_idx[(size_t)frow * p.cand_ld + slot + k] = ti[k];
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) { tv[k] = -3.0e38f; ti[k] = 0; }
          cur_m = mt;
        }
      }
      const int m0 = (tile / p.n_n_tiles) * (BM * NCTA) + (int)rank * BM;
      const int n0 = (tile % p.n_n_tiles) * p.BN;
      const int row = m0 + r;
      const int buf = t_local & 1;
      const uint32_t use = (uint32_t)(t_local >> 1);
      if (HAS_IN && elected && n_pan > 0) {
        // fetch the tile's first R panel while its main loop still runs; the panel is free once the stores
        // issued from it have read it
        tc::tma_store_wait_read<0>();
        tc::mbar_expect_tx(my_in_bar, IN_BYTES);
        tc::tma_load_2d(pan, &tmR, my_in_bar, n0 + g_col, m0);
        if (EPI == E_DW_SGD) tc::tma_load_2d(pan2, &tmF, my_in_bar, n0 + g_col, m0);
      }
      if (!tc::mbar_wait(tmem_full_bar + buf, use & 1, aborted, p.status, tc::SITE_TMEM_FULL, item)) *s_abort = 1;
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      if (*s_abort) break;                                   // the same answer in every epilogue warp
      tc::tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_STRIDE + (uint32_t)g_col;
      if (STAGED && n_pan > 0) {
        {
          const int pcol = n0 + g_col;                       // first column of this group's panel
          if (HAS_IN) {
            if (!tc::mbar_wait(my_in_bar, in_count & 1, aborted, p.status, tc::SITE_FULL, 2000 + g)) *s_abort = 1;
            ++in_count;
          } else {
            if (elected) tc::tma_store_wait_read<0>();       // the buffer is free once the previous store has read it
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          }
          uint4 keep2[EPI == E_BIAS_GELU ? 8 : 1];           // BIAS_GELU: the second output, packed, until the first has left
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {                   // two 32-column accumulator fragments per panel
            float v[32];
            tc::tmem_ld32(tbase + 32 * hc, v);
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              const int chunk = 4 * hc + j8;
              const int c = pcol + 8 * chunk;
              uint4* slot = reinterpret_cast<uint4*>(pan + panel_off(r, chunk));
              float* a = &v[8 * j8];
              float o[8];
              if (EPI == E_STORE) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = a[j];
              } else if (EPI == E_SIGMOID_POS) {
                if (p.loss_acc != nullptr && row < p.M) {
                  // sampled loss (dl_base.py:579-583): softplus of every logit here; minus the logits at the positives
                  // by a separate small kernel
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (c + j < p.N) loss += fmaxf(a[j], 0.f) + log1pf(__expf(-fabsf(a[j])));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = (c + j < p.N) ? 1.f / (1.f + __expf(-a[j])) : 0.f;
              } else if (EPI == E_BIAS_GELU) {
                float b[8];
                if (c < p.N) unpack8<T>(__ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.bias) + c)), b);
                else {
#pragma unroll
                  for (int j = 0; j < 8; ++j) b[j] = 0.f;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  o[j] = round_through<T>(a[j] + b[j]);      // the backward pass differentiates at the stored value
                  a[j] = gelu_f(o[j]);                       // second output, staged after the first has left
                }
              } else if (EPI == E_BIAS_DROPOUT_RESID) {
                float b[8], res[8];
                if (c < p.N) unpack8<T>(__ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.bias) + c)), b);
                else {
#pragma unroll
                  for (int j = 0; j < 8; ++j) b[j] = 0.f;
                }
                unpack8<T>(*slot, res);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float t = a[j] + b[j];
                  if (p.p > 0.f) t = keep(seed, p.stream, (uint32_t)(row * p.N + c + j), p.p) ? t * inv_keep : 0.f;
                  o[j] = res[j] + t;
                }
              } else if (EPI == E_ADD) {
                float res[8];
                unpack8<T>(*slot, res);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = a[j] + res[j];
              } else if (EPI == E_DW_SGD) {
                // momentum SGD on the tile: m = mo m + (dW + wd w), w -= lr m, with m rounded to 16 bit first
                uint4* slot2 = reinterpret_cast<uint4*>(pan2 + panel_off(r, chunk));
                float w[8], mm[8];
                unpack8<T>(*slot, w);
                unpack8<T>(*slot2, mm);
                const float lr = p.hp[HP_LR_XFC];
                const uint32_t sr_seed = reinterpret_cast<const uint32_t*>(p.hp)[HP_SEED];
                const uint32_t e = (uint32_t)row * (uint32_t)p.ldW + (uint32_t)c;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  mm[j] = round_through<T>(p.mo * mm[j] + (a[j] + p.wd * w[j]));
                  const float nw = w[j] - lr * mm[j];
                  o[j] = p.stochastic_round ? sr_round<T>(nw, mix32(sr_seed, 0x5152u, e + j)) : nw;
                }
                *slot2 = pack8<T>(mm);
              } else {   // E_GELU_BWD: rows past M read F = 0 and a zero accumulator, so they add nothing to the sums
                float f[8];
                unpack8<T>(*slot, f);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  o[j] = round_through<T>(a[j] * gelu_grad_f(f[j]));
                  a[j] = o[j];
                }
              }
              *slot = pack8<T>(o);
              if (EPI == E_BIAS_GELU) keep2[EPI == E_BIAS_GELU ? chunk : 0] = pack8<T>(a);
            }
            if (EPI == E_GELU_BWD && p.colacc != nullptr) {
              const float cs = warp_colsum32(v, lane);       // lane L holds the sum of column L of the fragment
              const int c = pcol + 32 * hc + lane;
              if (c < p.N) atomicAdd(p.colacc + (size_t)(blockIdx.x % kColReplicas) * p.col_tot + p.col_off + c, cs);
            }
          }
          if (EPI == E_SIGMOID_POS && p.pos_labels != nullptr) {
            // subtract 1 at the tile's positives while the tile is still in shared memory: entries of the label-sorted
            // list whose label is one of this CTA's 128 rows and whose batch row is one of the panel's 64 columns
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");      // every row of the panel is written
            const int nnz = *p.nnz_ptr;
            const int lab_lo = p.label0 + m0;
            const int lab_hi = p.label0 + min(m0 + BM, p.M);
            int lo = 0, hi = nnz;
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (p.pos_labels[mid] < lab_lo) lo = mid + 1; else hi = mid; }
            const int e0 = lo;
            hi = nnz;
            while (lo < hi) { const int mid = (lo + hi) >> 1; if (p.pos_labels[mid] < lab_hi) lo = mid + 1; else hi = mid; }
            const int e1 = lo;
            for (int e = e0 + (int)(threadIdx.x - 64 - 128 * g); e < e1; e += 128) {
              const int bcol = p.pos_rows[e] - pcol;
              if (bcol >= 0 && bcol < 64 && pcol + bcol < p.N) {
                const int prow = p.pos_labels[e] - lab_lo;
                T* cell = reinterpret_cast<T*>(pan + panel_off(prow, bcol >> 3)) + (bcol & 7);
                *cell = from_f<T>(to_f(*cell) - 1.f);      // duplicates are removed by the collator: one writer per cell
              }
            }
          }
          tc::fence_proxy_async();                 // generic-proxy writes of the panel before the async-proxy store
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          if (elected) {
            tc::tma_store_2d(EPI == E_BIAS_GELU ? &tmF : &tmC, pan, pcol, m0);
            if (EPI == E_DW_SGD) tc::tma_store_2d(&tmF, pan2, pcol, m0);
            tc::tma_store_commit();
          }
          if (EPI == E_BIAS_GELU) {
            // second output through the same panel: C = gelu(F), held in the fragment registers
            if (elected) tc::tma_store_wait_read<0>();
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
#pragma unroll
            for (int chunk = 0; chunk < 8; ++chunk)
              *reinterpret_cast<uint4*>(pan + panel_off(r, chunk)) = keep2[EPI == E_BIAS_GELU ? chunk : 0];
            tc::fence_proxy_async();
            asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
            if (elected) {
              tc::tma_store_2d(&tmC, pan, pcol, m0);
              tc::tma_store_commit();
            }
          }
        }
      }
      if (EPI == E_TOPK) {
        const uint32_t ttk = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_STRIDE + (uint32_t)(g * ucols);
        {
          for (int cc = 0; u_active && cc < ucols; cc += 32) {
            float v[32];
            tc::tmem_ld32(ttk + cc, v);
            const int c0 = n0 + g * ucols + cc;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float x = v[j];
              if (x > tv[7] && c0 + j < p.N) {           // strict: of equal values the lower column stays
                tv[7] = x; ti[7] = c0 + j;
#pragma unroll
                for (int k = 7; k > 0; --k) {
                  if (tv[k] > tv[k - 1]) {
                    const float a = tv[k]; tv[k] = tv[k - 1]; tv[k - 1] = a;
                    const int b = ti[k]; ti[k] = ti[k - 1]; ti[k - 1] = b;
                  }
                }
              }
            }
          }
        }
      }
      if (EPI == E_DX) {
        const float scale = p.hp[HP_SCALE];
        const uint32_t tdx = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_STRIDE + (uint32_t)(g * ucols);
        for (int c0 = 0; u_active && c0 < ucols; c0 += 32) {
          float v[32];
          tc::tmem_ld32(tdx + c0, v);
          const int col0 = n0 + g * ucols + c0;
          if (row < p.M) {
            float* d = p.dX + (size_t)row * p.ldX + col0;
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4)
              if (col0 + 4 * j4 < p.N)
                red_add_f32x4(d + 4 * j4, v[4 * j4] * scale, v[4 * j4 + 1] * scale, v[4 * j4 + 2] * scale, v[4 * j4 + 3] * scale);
          }
        }
      }
      if (EPI == E_SPLITK) {
        const uint32_t tsk = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)buf * ACC_STRIDE + (uint32_t)(g * ucols);
        for (int c0 = 0; u_active && c0 < ucols; c0 += 32) {
          float v[32];
          tc::tmem_ld32(tsk + c0, v);
          const int c_in_tile = g * ucols + c0;
          const int col0 = n0 + c_in_tile;
          if (row < p.M) {
            if (p.splits == 1) {
#pragma unroll
              for (int j8 = 0; j8 < 4; ++j8)
                if (col0 + 8 * j8 < p.N)
                  *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.C) + (size_t)row * p.ldc + col0 + 8 * j8) = pack8<T>(v + 8 * j8);
            } else {
              float* s = p.sk_scratch + (size_t)tile * (BM * NCTA * p.BN) + (size_t)((int)rank * BM + r) * p.BN + c_in_tile;
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4)
                if (col0 + 4 * j4 < p.N) red_add_f32x4(s + 4 * j4, v[4 * j4], v[4 * j4 + 1], v[4 * j4 + 2], v[4 * j4 + 3]);
            }
          }
        }
      }
      // every tcgen05.ld of this item has completed (tmem_ld32 waits): hand the accumulator back to the MMA warp
      tc::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (NCTA == 2) tc::mbar_arrive_leader(tmem_empty_bar + buf); else tc::mbar_arrive(tmem_empty_bar + buf);
      }
      if (EPI == E_SPLITK && p.splits > 1) {
        // split-K fix-up: the CTA that adds the last partial of its half of a tile converts the sum and re-zeroes
        // the scratch (each CTA of a pair counts its own half)
        unsigned* cnt = p.sk_counters + (size_t)tile * NCTA + rank;
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 64) *s_last = (atomicAdd(cnt, 1u) == (unsigned)(p.splits - 1)) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        if (*s_last) {
          // this CTA's 128 x BN block of the tile's scratch is contiguous: walk it with coalesced 16-byte accesses,
          // several loads in flight per thread
          __threadfence();
          T* C = reinterpret_cast<T*>(p.C);
          float4* blk = reinterpret_cast<float4*>(p.sk_scratch + (size_t)tile * (BM * NCTA * p.BN) + (size_t)((int)rank * BM) * p.BN);
          const int n4 = BM * p.BN / 4;
          const int bn4 = p.BN / 4;
          const int et = (int)threadIdx.x - 64;
          for (int base = et; base < n4; base += EPI_THREADS * 4) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i4 = base + EPI_THREADS * u;
              x[u] = i4 < n4 ? __ldcg(blk + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int i4 = base + EPI_THREADS * u;
              if (i4 < n4) {
                __stcg(blk + i4, make_float4(0.f, 0.f, 0.f, 0.f));
                const int rr = i4 / bn4, cc = (i4 - rr * bn4) * 4;
                const int grow = m0 + rr, gcol = n0 + cc;
                if (grow < p.M && gcol < p.N) {
                  uint2 o;
                  T* e = reinterpret_cast<T*>(&o);
                  e[0] = from_f<T>(x[u].x); e[1] = from_f<T>(x[u].y); e[2] = from_f<T>(x[u].z); e[3] = from_f<T>(x[u].w);
                  *reinterpret_cast<uint2*>(C + (size_t)grow * p.ldc + gcol) = o;
                }
              }
            }
          }
          if (threadIdx.x == 64) *cnt = 0u;
        }
      }
    }
    if (STAGED && elected) tc::tma_store_wait_read<0>();   // the stores have read shared memory; they complete before the grid does
    if (EPI == E_SIGMOID_POS && p.loss_acc != nullptr) {
      loss = warp_sum(loss);
      if (lane == 0 && loss != 0.f) atomicAdd(p.loss_acc, loss);
    }
    if (EPI == E_DX && p.done_counter != nullptr) {
      // reduce-scatter epilogue: the last CTA of this rank's dX GEMM tells every rank that the partial sums in this
      // rank's buffer are complete
      __threadfence_system();
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      if (threadIdx.x == 64) {
        if (atomicAdd(p.done_counter, 1u) == gridDim.x - 1) {
          *p.done_counter = 0u;
          __threadfence_system();
          const uint32_t tagv = *p.step_ptr;
          for (int q = 0; q < p.n_peers; ++q) st_release_sys(reinterpret_cast<uint32_t*>(p.peer_flags[q]) + p.flag_index, tagv);
        }
      }
    }
    if (EPI == E_TOPK && cur_m >= 0 && u_active) {
      const int frow = cur_m * (BM * NCTA) + (int)rank * BM + r;
      if (frow < p.M) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          p.cand_val[(size_t)frow * p.cand_ld + slot + k] = tv[k];
          p.cand_idx[(size_t)frow * p.cand_ld + slot + k] = ti[k];
        }
      }
    }
  }
  tc::tc_fence_before();
  __syncthreads();
  if (NCTA == 2) tc::cluster_sync_all();                   // the peer no longer reads this CTA's memory or barriers
  if (warp == 1) {
    tc::tc_fence_after();
    if (NCTA == 2) tc::tmem_dealloc_pair(tmem_base, TMEM_COLS); else tc::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace eg
}  // namespace rb

// ------------------------------------------------------------------------------------ LayerNorm of a stored input
// y = LN(pre) with the row statistics kept for the backward pass; `pre` was written by the BIAS_DROPOUT_RESID
// epilogue.  One warp per row, 16-byte accesses.
namespace rb {
namespace eg {
template <typename T, int NV>
__global__ void __launch_bounds__(128) ln_fwd_kernel(const T* __restrict__ pre, const T* __restrict__ gamma,
                                                     const T* __restrict__ beta, T* __restrict__ y,
                                                     float* __restrict__ mean, float* __restrict__ rstd, int rows, int H,
                                                     float eps) {
  grid_dep_wait();            // launched with launch_pdl: nothing above touches global memory
  grid_dep_launch();          // the kernel that follows may start its set-up now; it waits for this grid before reading
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

struct Maps { CUtensorMap a, b, c, r, f; };

// Programmatic dependent launch (a kernel's set-up overlaps the previous kernel's tail): on by default.
RB_API void rb_enc_gemm_set_pdl(int on) { pdl_flag() = on ? 1 : 0; }

template <typename T, int LAYOUT, int EPI, int NCTA>
static int launch_enc_gemm(const Maps& m, const Params& p, int units, cudaStream_t st) {
  static bool attr_set = false;
  auto k = enc_gemm_kernel<T, LAYOUT, EPI, NCTA>;
  constexpr int smem = Cfg<EPI>::kSmem;
  if (!attr_set) {
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -5;
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(NCTA * units, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (NCTA == 2) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (pdl_flag()) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, k, m.a, m.b, m.c, m.r, m.f, p);
  return e == cudaSuccess ? 0 : (int)e;
}

template <typename T, int NCTA>
static int dispatch_enc_gemm(int layout, int epi, const Maps& m, const Params& p, int units, cudaStream_t st) {
  if (layout == L_NT) {
    if (epi == E_STORE) return launch_enc_gemm<T, L_NT, E_STORE, NCTA>(m, p, units, st);
    if (epi == E_BIAS_GELU) return launch_enc_gemm<T, L_NT, E_BIAS_GELU, NCTA>(m, p, units, st);
    if (epi == E_BIAS_DROPOUT_RESID) return launch_enc_gemm<T, L_NT, E_BIAS_DROPOUT_RESID, NCTA>(m, p, units, st);
    if (epi == E_TOPK) return launch_enc_gemm<T, L_NT, E_TOPK, NCTA>(m, p, units, st);
    if (epi == E_SIGMOID_POS) return launch_enc_gemm<T, L_NT, E_SIGMOID_POS, NCTA>(m, p, units, st);
  } else if (layout == L_NN) {
    if (epi == E_STORE) return launch_enc_gemm<T, L_NN, E_STORE, NCTA>(m, p, units, st);
    if (epi == E_ADD) return launch_enc_gemm<T, L_NN, E_ADD, NCTA>(m, p, units, st);
    if (epi == E_GELU_BWD) return launch_enc_gemm<T, L_NN, E_GELU_BWD, NCTA>(m, p, units, st);
    if (epi == E_DW_SGD) return launch_enc_gemm<T, L_NN, E_DW_SGD, NCTA>(m, p, units, st);
  } else if (layout == L_TN) {
    if (epi == E_SPLITK) return launch_enc_gemm<T, L_TN, E_SPLITK, NCTA>(m, p, units, st);
    if (epi == E_DX) return launch_enc_gemm<T, L_TN, E_DX, NCTA>(m, p, units, st);
  }
  return -4;
}

// Tile shape and K-splits from a cost model calibrated on B200 (clocks per CTA):
//   * a k block costs max(MMA time = 2 BN, operand bytes of the CTA / fetch rate); with every SM busy an SM sustains
//     about 29 bytes per clock from L2 (the L2-to-SM fabric, about 8 TB/s in total, is the shared limit), with
//     fewer SMs busy proportionally more, down to a floor of about 3900 clocks of load latency divided by the
//     number of ring stages (192 KB / stage size: 4 to 8);
//   * work is spread over the units (SMs, or SM pairs) in rounds;
//   * about 3000 clocks of start-up per kernel (TMEM allocation, barrier set-up, first load);
//   * the epilogue of a CTA's last tile is exposed: per 64-column panel about 1200 clocks (store), 2400 (two
//     outputs), 2800 (a tile-shaped input fetched after the previous panel has left; the first panel's input is
//     fetched under the main loop);
//   * a K-split costs about 10000 clocks (partial sums through L2 atomics, the last CTA's conversion pass).
struct Plan { int ncta, bn, splits, tiles; };

static int g_max_units = 0;
// Experiments: cap the number of persistent workers (0 = one per SM / SM pair).
RB_API void rb_enc_gemm_set_max_units(int n) { g_max_units = n; }

static Plan make_plan(int layout, int epi, int M, int N, int K, int bn_forced, int ncta_forced) {
  const int sms = sm_count();
  const int kb = (K + BK - 1) / BK;
  Plan best{1, 128, 1, 1};
  double best_cost = -1.0;
  for (int ncta = 1; ncta <= 2; ++ncta) {
    if (ncta_forced && ncta != ncta_forced) continue;
    for (int bn = 256; bn >= 64; bn >>= 1) {
      if (bn_forced && bn != bn_forced) continue;
      if (ncta == 2 && bn < 128) continue;
      if (!bn_forced && bn > 64 && bn / 2 >= N) continue;            // a narrower tile already covers every column
      const int tiles = ((M + BM * ncta - 1) / (BM * ncta)) * ((N + bn - 1) / bn);
      const int units = sms / ncta;
      int max_splits = layout == L_TN ? (kb < 16 ? kb : 16) : 1;
      int first_split = 1;
      if (epi == E_DX) {                      // partial sums are reduced into the output directly: split as far as the units go
        first_split = units / tiles < 1 ? 1 : (units / tiles > kb ? kb : units / tiles);
        max_splits = first_split;
      }
      for (int splits = first_split; splits <= max_splits; splits = (splits == max_splits ? max_splits + 1 : splits * 2)) {
        const int kb_per = (kb + splits - 1) / splits;
        const int eff_splits = (kb + kb_per - 1) / kb_per;
        if (eff_splits != splits && splits > 1 && epi != E_DX) continue;
        const long items = (long)tiles * eff_splits;
        const long rounds = (items + units - 1) / units;
        const double busy = (double)(items < units ? items : units) * ncta / sms;      // fraction of the SMs at work
        const double bytes = A_BYTES + (double)(bn / ncta) * BK * 2;
        double t_kb = bytes / (29.0 / (busy > 0.25 ? busy : 0.25));
        const int stages = (int)(ring_bytes(epi) / bytes) < MAX_STAGES ? (int)(ring_bytes(epi) / bytes) : MAX_STAGES;
        if (t_kb < 3900.0 / stages) t_kb = 3900.0 / stages;          // load latency over the ring depth
        if (t_kb < 2.0 * bn) t_kb = 2.0 * bn;
        const int n_pan = 1;                                         // one staging panel per group and tile
        double tail;
        if (epi == E_SPLITK || epi == E_TOPK || epi == E_DX) tail = 800.0 * n_pan;
        else if (epi == E_STORE) tail = 1200.0 * n_pan;
        else if (epi == E_BIAS_GELU) tail = 2400.0 * n_pan;
        else tail = 1200.0 + 2800.0 * (n_pan - 1);
        const double cost = 3000.0 + rounds * (kb_per * t_kb) + tail + (eff_splits > 1 && epi != E_DX ? 10000.0 : 0.0);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = Plan{ncta, bn, eff_splits, tiles}; }
      }
    }
  }
  return best;
}

// What rb_enc_gemm will use for (M, N, K): tile shape, K-splits for layout TN, and the sizes of the split-K
// scratch (floats) and counters (words) it needs when splits > 1.
RB_API int rb_enc_gemm_plan(int layout, int epi, int M, int N, int K, int bn_forced, int ncta_forced, int* ncta_out,
                            int* bn_out, int* splits_out, long long* scratch_floats, int* counter_words) {
  const Plan pl = make_plan(layout, epi, M, N, K, bn_forced, ncta_forced);
  *ncta_out = pl.ncta; *bn_out = pl.bn; *splits_out = pl.splits;
  *scratch_floats = (long long)pl.tiles * BM * pl.ncta * pl.bn;
  *counter_words = pl.tiles * pl.ncta;
  return 0;
}

// C = op(A) op(B) with a fused epilogue; see the head of this file.  Leading dimensions in elements.
//   layout 0 (NT): A[M, lda>=K], B[N, ldb>=K];  1 (NN): A[M, lda>=K], B[K, ldb>=N];  2 (TN): A[K, lda>=M], B[K, ldb>=N]
//   dtype: RB_BF16 or RB_F16 (operands, C, bias, R and F all have it; accumulation is fp32)
//   R [M, ldr]: residual (BIAS_DROPOUT_RESID, ADD) or stored pre-activation (GELU_BWD); F [M, ldf]: pre-activation
//   output (BIAS_GELU).  Layout TN with more than one K-split needs sk_scratch / sk_counters of the sizes
//   rb_enc_gemm_plan reports (zero on entry, left zero).  bn_forced / ncta_forced: 0 = choose.
// Returns 0, or -3 for an unsupported shape (the caller then uses the library GEMM).
RB_API int rb_enc_gemm(int dtype, int layout, int epi, const void* A, const void* B, void* C, int M, int N, int K, int lda,
                       int ldb, int ldc, const void* bias, const void* R, int ldr, void* F, int ldf, float p_drop,
                       const int* seed, unsigned stream_id, float* colacc, int col_tot, int col_off, float* sk_scratch,
                       unsigned* sk_counters, int bn_forced, int ncta_forced, int* status, cudaStream_t st) {
  if (dtype != RB_BF16 && dtype != RB_F16) return -1;
  if (M < 1 || N < 1 || K < 1 || N % 8 || lda % 8 || ldb % 8 || ldc % 8 || ldr % 8 || ldf % 8) return -3;
  if (layout == L_TN && M % 8) return -3;
  if ((epi == E_BIAS_GELU || epi == E_BIAS_DROPOUT_RESID) && bias == nullptr) return -3;
  if ((epi == E_BIAS_DROPOUT_RESID || epi == E_ADD || epi == E_GELU_BWD) && R == nullptr) return -3;
  if (epi == E_BIAS_GELU && F == nullptr) return -3;
  if (epi == E_BIAS_DROPOUT_RESID && p_drop > 0.f && seed == nullptr) return -3;
  const bool bf16 = dtype == RB_BF16;
  const Plan pl = make_plan(layout, epi, M, N, K, bn_forced, ncta_forced);
  const int BN = pl.bn, b_rows = BN / pl.ncta;
  Maps m;
  int rc;
  if (layout == L_TN) rc = tc::make_tmap_2d(&m.a, A, K, M, lda, 64, 64, bf16);
  else rc = tc::make_tmap_2d(&m.a, A, M, K, lda, 64, BM, bf16);
  if (rc) return rc;
  if (layout == L_NT) rc = tc::make_tmap_2d(&m.b, B, N, K, ldb, 64, b_rows, bf16);
  else rc = tc::make_tmap_2d(&m.b, B, K, N, ldb, 64, 64, bf16);
  if (rc) return rc;
  // output / input panels: [128 rows x 64 columns] boxes of the row-major [M, N] matrices
  rc = tc::make_tmap_2d(&m.c, C, M, N, ldc, 64, BM, bf16);
  if (rc) return rc;
  m.r = m.c;
  m.f = m.c;
  if (R != nullptr && (rc = tc::make_tmap_2d(&m.r, R, M, N, ldr, 64, BM, bf16)) != 0) return rc;
  if (F != nullptr && (rc = tc::make_tmap_2d(&m.f, F, M, N, ldf, 64, BM, bf16)) != 0) return rc;
  Params p{};
  p.M = M; p.N = N; p.BN = BN;
  p.n_m_tiles = (M + BM * pl.ncta - 1) / (BM * pl.ncta); p.n_n_tiles = (N + BN - 1) / BN;
  p.kb_total = (K + BK - 1) / BK;
  p.splits = pl.splits;
  p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  if (p.splits > 1 && (sk_scratch == nullptr || sk_counters == nullptr)) return -3;
  p.C = C; p.ldc = ldc; p.bias = bias;
  p.p = p_drop; p.seed = seed; p.stream = stream_id;
  p.colacc = colacc; p.col_tot = col_tot; p.col_off = col_off;
  p.sk_scratch = sk_scratch; p.sk_counters = sk_counters; p.status = status;
  const int n_items = p.n_m_tiles * p.n_n_tiles * p.splits;
  int max_units = sm_count() / pl.ncta;
  if (g_max_units > 0 && g_max_units < max_units) max_units = g_max_units;
  const int units = n_items < max_units ? n_items : max_units;
  if (pl.ncta == 2)
    rc = bf16 ? dispatch_enc_gemm<__nv_bfloat16, 2>(layout, epi, m, p, units, st) : dispatch_enc_gemm<__half, 2>(layout, epi, m, p, units, st);
  else
    rc = bf16 ? dispatch_enc_gemm<__nv_bfloat16, 1>(layout, epi, m, p, units, st) : dispatch_enc_gemm<__half, 1>(layout, epi, m, p, units, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// Prediction: candidates for the top-k (k <= 8) of every row of X W^T without materialising the product.
//   X [B, ldx >= D], W [Ls, ldw >= D] (16-bit, same dtype); cand_val / cand_idx [B, cand_ld] with
//   cand_ld >= rb_xfc_topk8_width(): every (CTA, epilogue group) writes the 8 best (value, column of W) it met in
//   the row into its own 8 entries; entries nobody writes must have been pre-filled with -inf by the caller.
// The k best of a row's candidates are the k best of the row (k <= 8).
RB_API int rb_xfc_topk8_width(void) { return sm_count() * EGROUPS * 8; }

RB_API int rb_xfc_topk8(int dtype, const void* X, const void* W, int B, int Ls, int D, int ldx, int ldw, float* cand_val,
                        int* cand_idx, int cand_ld, int* status, cudaStream_t st) {
  if (dtype != RB_BF16 && dtype != RB_F16) return -1;
  if (B < 1 || Ls < 1 || D < 1 || ldx % 8 || ldw % 8 || cand_ld < rb_xfc_topk8_width()) return -3;
  const bool bf16 = dtype == RB_BF16;
  const Plan pl = make_plan(L_NT, E_TOPK, B, Ls, D, 0, 0);
  const int BN = pl.bn, b_rows = BN / pl.ncta;
  Maps m;
  int rc = tc::make_tmap_2d(&m.a, X, B, D, ldx, 64, BM, bf16);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&m.b, W, Ls, D, ldw, 64, b_rows, bf16);
  if (rc) return rc;
  m.c = m.a; m.r = m.a; m.f = m.a;
  Params p{};
  p.M = B; p.N = Ls; p.BN = BN;
  p.n_m_tiles = (B + BM * pl.ncta - 1) / (BM * pl.ncta); p.n_n_tiles = (Ls + BN - 1) / BN;
  p.kb_total = (D + BK - 1) / BK; p.splits = 1; p.kb_per_split = p.kb_total;
  p.cand_val = cand_val; p.cand_idx = cand_idx; p.cand_ld = cand_ld; p.status = status;
  const long n_items = (long)p.n_m_tiles * p.n_n_tiles;
  const int max_units = sm_count() / pl.ncta;
  const int units = n_items < max_units ? (int)n_items : max_units;
  rc = pl.ncta == 2
           ? (bf16 ? dispatch_enc_gemm<__nv_bfloat16, 2>(L_NT, E_TOPK, m, p, units, st) : dispatch_enc_gemm<__half, 2>(L_NT, E_TOPK, m, p, units, st))
           : (bf16 ? dispatch_enc_gemm<__nv_bfloat16, 1>(L_NT, E_TOPK, m, p, units, st) : dispatch_enc_gemm<__half, 1>(L_NT, E_TOPK, m, p, units, st));
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

template <int DUMMY = 0>
static int launch_planned(const Plan& pl, bool bf16, int layout, int epi, const Maps& m, Params& p, int K, cudaStream_t st) {
  p.BN = pl.bn;
  p.n_m_tiles = (p.M + BM * pl.ncta - 1) / (BM * pl.ncta); p.n_n_tiles = (p.N + pl.bn - 1) / pl.bn;
  p.kb_total = (K + BK - 1) / BK;
  p.splits = pl.splits;
  p.kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
  const long n_items = (long)p.n_m_tiles * p.n_n_tiles * p.splits;
  int max_units = sm_count() / pl.ncta;
  if (g_max_units > 0 && g_max_units < max_units) max_units = g_max_units;
  const int units = n_items < max_units ? (int)n_items : max_units;
  return pl.ncta == 2
             ? (bf16 ? dispatch_enc_gemm<__nv_bfloat16, 2>(layout, epi, m, p, units, st) : dispatch_enc_gemm<__half, 2>(layout, epi, m, p, units, st))
             : (bf16 ? dispatch_enc_gemm<__nv_bfloat16, 1>(layout, epi, m, p, units, st) : dispatch_enc_gemm<__half, 1>(layout, epi, m, p, units, st));
}

// Classifier logits + gradient on the persistent GEMM: Gt[Lc, ldG] = sigmoid(W X^T) - Y for the fp16 label chunk
// W[Lc, D] and the gathered embeddings X[B, D]; columns B .. ldG of Gt are written as zeros.  Positives: label-sorted
// (row, label) pairs, labels numbered from label0 at row 0 of W; they are subtracted in shared memory before the tile
// is stored.  wait_flags != null: the loads wait until flags[0 .. wait_n) have reached *step_ptr (all-gather landed).
// Replaces, in the reference, torch.matmul + sigmoid_ + index_put_ (dl_base.py:572, 593-594) / the CUTLASS
// sigmoid-GEMM (xfc_gemm_kernel.cu:59-100).
RB_API int rb_xfc_logits_grad_v2(const void* W, int Lc, int D, const void* X, int B, void* Gt, int ldG, const int* pos_rows,
                                 const int* pos_labels, const int* nnz_ptr, int label0, const unsigned* wait_flags,
                                 int wait_n, const unsigned* step_ptr, float* loss_acc, int* status, cudaStream_t st) {
  if (D % 8 || ldG % 8 || Lc < 1 || B < 1 || ldG < B) return -3;
  const Plan pl = make_plan(L_NT, E_SIGMOID_POS, Lc, B, D, 0, 0);
  Maps m;
  int rc = tc::make_tmap_2d(&m.a, W, Lc, D, D, 64, BM, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&m.b, X, B, D, D, 64, pl.bn / pl.ncta, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&m.c, Gt, Lc, ldG, ldG, 64, BM, false);
  if (rc) return rc;
  m.r = m.c; m.f = m.c;
  Params p{};
  p.M = Lc; p.N = B; p.status = status;
  p.pos_rows = pos_rows; p.pos_labels = pos_labels; p.nnz_ptr = nnz_ptr; p.label0 = label0;
  p.wait_flags = wait_flags; p.wait_n = wait_n; p.step_ptr = step_ptr; p.loss_acc = loss_acc;
  rc = launch_planned(pl, false, L_NT, E_SIGMOID_POS, m, p, D, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// dX[B, D] += hp[SCALE] * Gt^T W over the label chunk (fp32, vector reductions; dX zeroed before the first chunk).
// done_counter != null: the last CTA stores *step_ptr into word flag_index of every peer's flag array.
RB_API int rb_xfc_dx_v2(const void* Gt, int ldG, const void* W, int Lc, int D, int B, float* dX, const float* hp,
                        unsigned* done_counter, void* const* peer_flags, int n_peers, int flag_index,
                        const unsigned* step_ptr, int* status, cudaStream_t st) {
  if (D % 8 || ldG % 8 || Lc < 1 || B < 1 || n_peers > 16) return -3;
  const Plan pl = make_plan(L_TN, E_DX, B, D, Lc, 0, 0);
  Maps m;
  int rc = tc::make_tmap_2d(&m.a, Gt, Lc, B, ldG, 64, 64, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&m.b, W, Lc, D, D, 64, 64, false);
  if (rc) return rc;
  m.c = m.a; m.r = m.a; m.f = m.a;
  Params p{};
  p.M = B; p.N = D; p.status = status;
  p.dX = dX; p.ldX = D; p.hp = hp;
  if (done_counter != nullptr) {
    p.done_counter = done_counter; p.n_peers = n_peers; p.flag_index = flag_index; p.step_ptr = step_ptr;
    for (int q = 0; q < n_peers; ++q) p.peer_flags[q] = peer_flags[q];
  }
  rc = launch_planned(pl, false, L_TN, E_DX, m, p, Lc, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
  return 0;
}

// Classifier weight update on the persistent GEMM: dW = Gt X over the batch (never stored), then momentum SGD on the
// [128 x 64] tiles of W and Mom [Lc, D] (fp16) in shared memory: both tiles come in by TMA under the main loop and
// leave by TMA; lr and the rounding seed are read from hp on the device.
// Replaces, in the reference, the fused dW GEMM + SGD epilogue (xfc_gemm_kernel.cu:102-151).
RB_API int rb_xfc_dw_sgd_v2(const void* Gt, int ldG, const void* X, int B, void* W, void* Mom, int Lc, int D,
                            const float* hp, float mo, float wd, int stochastic_round, int bn_forced, int ncta_forced,
                            int* status, cudaStream_t st) {
  if (D % 8 || ldG % 8 || Lc < 1 || B < 1) return -3;
  const Plan pl = make_plan(L_NN, E_DW_SGD, Lc, D, B, bn_forced, ncta_forced);
  Maps m;
  int rc = tc::make_tmap_2d(&m.a, Gt, Lc, B, ldG, 64, BM, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&m.b, X, B, D, D, 64, 64, false);
  if (rc) return rc;
  rc = tc::make_tmap_2d(&m.c, W, Lc, D, D, 64, BM, false);
  if (rc) return rc;
  m.r = m.c;
  rc = tc::make_tmap_2d(&m.f, Mom, Lc, D, D, 64, BM, false);
  if (rc) return rc;
  Params p{};
  p.M = Lc; p.N = D; p.status = status;
  p.hp = hp; p.mo = mo; p.wd = wd; p.stochastic_round = stochastic_round; p.ldW = D;
  rc = launch_planned(pl, false, L_NN, E_DW_SGD, m, p, B, st);
  if (rc) return rc;
  RB_LAUNCH_CHECK();
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
    case RB_F32: { using T = float; EG_DISPATCH_NV(H, (launch_pdl(ln_fwd_kernel<T, NV>, dim3(blocks), dim3(128), 0, st, (const T*)pre, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, H, eps))); break; }
    case RB_BF16: { using T = __nv_bfloat16; EG_DISPATCH_NV(H, (launch_pdl(ln_fwd_kernel<T, NV>, dim3(blocks), dim3(128), 0, st, (const T*)pre, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, H, eps))); break; }
    case RB_F16: { using T = __half; EG_DISPATCH_NV(H, (launch_pdl(ln_fwd_kernel<T, NV>, dim3(blocks), dim3(128), 0, st, (const T*)pre, (const T*)gamma, (const T*)beta, (T*)y, mean, rstd, rows, H, eps))); break; }
    default: return -1;
  }
  RB_LAUNCH_CHECK();
  return 0;
}
