// Collectives over NVLink peer memory, written as plain kernels that load from / store to the other
// GPUs' buffers (P2P mappings of a symmetric allocation) and synchronise through step-tagged flags:
//
//   ag_push         classifier-input dropout + fp16 cast of this rank's embeddings, stored straight into
//                   every rank's gathered-X buffer, then "rows of rank r are in" flags     (signals)
//                   -> the logits GEMM's producer warp waits for the flags (xfc.cu)        (waits)
//   rs_pull         waits for every rank's "my dX partial is complete" flag (raised by the last CTA of
//                   its dX GEMM, xfc.cu), sums this rank's rows over all ranks' partials and applies the
//                   dropout backward                                                       (waits)
//   signal          raises one flag on every rank after a system-scope fence               (signals)
//   grad_allreduce  two-shot all-reduce of a range of the flat encoder-gradient buffer: this rank sums
//                   its 1/G slice over all ranks (fp32 accumulation, non-finite detection) and stores the
//                   result into every rank's buffer                         (waits on A, signals B)
//   wait_flags      waits for "all ranks have pushed their slices" and folds the non-finite words into
//                   the found-inf flag                                                     (waits)
//   step_inc        advances the device-resident step counter the tags are derived from
//
// They replace NCCL all_gather / all_reduce / the DDP bucket all-reduce of the reference
// (dl_base.py:547-555, 617, main.py:161).  For a given flag class a kernel either signals or waits,
// never both, so emulated ranks can be run one after another on a single GPU in tests.  Every wait is
// bounded: on expiry it records a status word and the kernel finishes normally.  Buffers written by
// peers are double-buffered by step parity on the host side.
#include <cstring>
#include "peer.cuh"

namespace rb {

// All threads of the block learn whether flags[0..n) have all reached `want`.
__device__ __forceinline__ bool block_wait_flags(const uint32_t* flags, int n, uint32_t want, int* status, int detail) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < n) {
    if (!wait_flag(flags + threadIdx.x, want, status, detail * 100 + (int)threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  return ok_s != 0;
}

__global__ void step_inc_kernel(uint32_t* step) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *step += 1u;
}

// ------------------------------------------------------------------------------------ all-gather push
// grid = (G, nblk).  Block (peer, j) writes its share of this rank's rows into `peer`'s X buffer.
__global__ void __launch_bounds__(256) ag_push_kernel(const float* __restrict__ e, int b, int D, float p,
                                                      const int* __restrict__ seed_ptr, uint32_t stream, PeerPtrs xbuf,
                                                      int row0, PeerPtrs flags, int flag_base, int my_rank, StepTag tag,
                                                      unsigned* __restrict__ counters) {
  const int peer = blockIdx.x;
  __half* dst = reinterpret_cast<__half*>(xbuf.p[peer]) + (size_t)row0 * D;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  const size_t n_vec = (size_t)b * D / 8;
  for (size_t i = (size_t)blockIdx.y * blockDim.x + threadIdx.x; i < n_vec; i += (size_t)gridDim.y * blockDim.x) {
    float v[8];
    load8(e + i * 8, v);
    if (p > 0.f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = keep(seed, stream, (uint32_t)(i * 8 + j), p) ? v[j] * inv_keep : 0.f;
    }
    store8(dst + i * 8, v);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counters + peer, 1u);
    if (done == gridDim.y - 1) {
      counters[peer] = 0u;
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[peer]) + flag_base + my_rank, tag.value());
    }
  }
}

// ------------------------------------------------------------------------------------ generic all-gather push
// grid = (G, nblk).  Block (peer, j) copies its share of this rank's n16 16-byte words into `peer`'s buffer at word
// offset slot16, then the last block per peer raises flag [flag_base + my_rank] there.  Used for the cross-rank merge
// of top-k candidates at prediction time (the reference: two NCCL all-gathers per batch, dl_base.py:774-775).
__global__ void __launch_bounds__(256) peer_gather_kernel(const uint4* __restrict__ src, long long n16, PeerPtrs dst,
                                                          long long slot16, PeerPtrs flags, int flag_base, int my_rank,
                                                          StepTag tag, unsigned* __restrict__ counters) {
  const int peer = blockIdx.x;
  uint4* out = reinterpret_cast<uint4*>(dst.p[peer]) + slot16;
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.y * blockDim.x)
    out[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counters + peer, 1u);
    if (done == gridDim.y - 1) {
      counters[peer] = 0u;
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(flags.p[peer]) + flag_base + my_rank, tag.value());
    }
  }
}

// ------------------------------------------------------------------------------------ reduce-scatter pull
// grid = rows of this rank; de[r, :] = dropout_bwd( sum_q partial_q[row0 + r, :] )
__global__ void __launch_bounds__(128) rs_pull_kernel(PeerPtrs partials, int G, int row0, int b, int D,
                                                      float* __restrict__ de, const uint32_t* __restrict__ my_flags,
                                                      StepTag tag, float p, const int* __restrict__ seed_ptr,
                                                      uint32_t stream, int* status) {
  const bool ok = block_wait_flags(my_flags, G, tag.value(), status, 2);
  const int r = blockIdx.x;
  if (r >= b) return;
  const uint32_t seed = p > 0.f ? (uint32_t)(*seed_ptr) : 0u;
  const float inv_keep = p > 0.f ? 1.f / (1.f - p) : 1.f;
  for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
      for (int q = 0; q < G; ++q) {
        const float* src = reinterpret_cast<const float*>(partials.p[q]) + (size_t)(row0 + r) * D + c;
        const uint4 raw = ld_sys_v4(src);
        acc.x += __uint_as_float(raw.x); acc.y += __uint_as_float(raw.y);
        acc.z += __uint_as_float(raw.z); acc.w += __uint_as_float(raw.w);
      }
    }
    if (p > 0.f) {
      const uint32_t base = (uint32_t)(r * D + c);
      acc.x = keep(seed, stream, base, p) ? acc.x * inv_keep : 0.f;
      acc.y = keep(seed, stream, base + 1, p) ? acc.y * inv_keep : 0.f;
      acc.z = keep(seed, stream, base + 2, p) ? acc.z * inv_keep : 0.f;
      acc.w = keep(seed, stream, base + 3, p) ? acc.w * inv_keep : 0.f;
    }
    *reinterpret_cast<float4*>(de + (size_t)r * D + c) = acc;
  }
}

// ------------------------------------------------------------------------------------ generic signal / wait
__global__ void signal_kernel(PeerPtrs flags, int G, int flag_base, int my_rank, StepTag tag) {
  __threadfence_system();
  if ((int)threadIdx.x < G)
    st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + flag_base + my_rank, tag.value());
}

// waits for flags[0..G) >= tag; then ORs the peers' non-finite words into hp[FOUND_INF] and clears them
__global__ void wait_flags_kernel(const uint32_t* my_flags, int G, StepTag tag, uint32_t* found_words, float* hp,
                                  int* status) {
  block_wait_flags(my_flags, G, tag.value(), status, 3);
  if (threadIdx.x == 0 && found_words != nullptr) {
    uint32_t any = 0;
    for (int q = 0; q < G; ++q) { any |= ld_acquire_sys(found_words + q); found_words[q] = 0u; }
    if (any) hp[HP_FOUND_INF] = 1.0f;
  }
}

// ------------------------------------------------------------------------------------ gradient all-reduce
// Range [lo, hi) of the flat gradient buffer (element offsets, multiples of 8).  This rank reduces the
// G-th part `my_rank` of the range and stores the sums into every rank's buffer.
template <typename T>
__global__ void __launch_bounds__(256) grad_allreduce_kernel(PeerPtrs grads, long long lo, long long hi, int G, int my_rank,
                                                             const uint32_t* __restrict__ my_flags_a, StepTag tag_a,
                                                             PeerPtrs flags, int flag_b_base, int found_base, StepTag tag_b,
                                                             unsigned* __restrict__ counter, int* status) {
  const bool ok = block_wait_flags(my_flags_a, G, tag_a.value(), status, 4);
  const long long n_vec = (hi - lo) / 8;
  const long long per = (n_vec + G - 1) / G;
  const long long v0 = min(n_vec, per * my_rank), v1 = min(n_vec, per * (my_rank + 1));
  bool bad = false;
  if (ok) {
    for (long long i = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < v1; i += (long long)gridDim.x * blockDim.x) {
      const size_t e = (size_t)(lo + i * 8);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int q = 0; q < G; ++q) {
        const uint4 raw = ld_sys_v4(reinterpret_cast<const T*>(grads.p[q]) + e);
        const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += to_f(h[j]);
      }
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int j = 0; j < 8; ++j) { bad |= !isfinite(acc[j]); o[j] = from_f<T>(acc[j]); }
      for (int q = 0; q < G; ++q) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(grads.p[q]) + e) = out;
    }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) {
    for (int q = 0; q < G; ++q) reinterpret_cast<uint32_t*>(flags.p[q])[found_base + my_rank] = 1u;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counter, 1u);
    if (done == gridDim.x - 1) {
      *counter = 0u;
      __threadfence_system();
      const uint32_t v = tag_b.value();
      for (int q = 0; q < G; ++q) st_release_sys(reinterpret_cast<uint32_t*>(flags.p[q]) + flag_b_base + my_rank, v);
    }
  }
}

// ------------------------------------------------------------------------------------ sharded optimizer
// Instead of all-reducing the gradients and running AdamW on all parameters on every rank, each rank
//   (A) sums ITS 1/G slice of the flat gradient over all ranks into a local fp32 buffer (reduce-scatter),
//       flags non-finite values to every rank and raises "slice reduced";
//   (B) after every rank's (A) is known to be done (so the found-inf decision is global), applies AdamW
//       to its slice of the fp32 master weights / moments and stores the new 16-bit weights of the slice
//       into EVERY rank's compute copy (all-gather of parameters), then raises "slice pushed".
// NVLink traffic equals that of the all-reduce it replaces; the AdamW traffic to HBM drops by 1/G.
// [v0, v1): the 8-element vectors of the flat buffer this rank reduces in this launch (its slice of the whole
// buffer, or its slice of one bucket when the reduction is overlapped with the backward pass); tag_a: value the
// peers' progress flags must have reached; flag_b_base < 0: no "slice reduced" signal after this launch.
template <typename T>
__global__ void __launch_bounds__(256) grad_reduce_scatter_kernel(PeerPtrs grads, long long v0, long long v1, int G,
                                                                  int my_rank, const uint32_t* __restrict__ my_flags_a,
                                                                  StepTag tag_a, StepTag tag, float* __restrict__ gsum,
                                                                  PeerPtrs flags, int flag_b_base, int found_base,
                                                                  unsigned* __restrict__ counter, int* status,
                                                                  const void* mc_grads) {
  const bool ok = block_wait_flags(my_flags_a, G, tag_a.value(), status, 5);
  bool bad = false;
  if (ok) {
    for (long long i = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < v1; i += (long long)gridDim.x * blockDim.x) {
      float acc[8];
      if (mc_grads != nullptr) {
        // in-switch reduction: one 16-byte load returns the sum of all ranks' 8 gradients
        const uint4 raw = multimem_ld_reduce_v4<T>(reinterpret_cast<const T*>(mc_grads) + i * 8);
        const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = to_f(h[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int q = 0; q < G; ++q) {
          const uint4 raw = ld_sys_v4(reinterpret_cast<const T*>(grads.p[q]) + i * 8);
          const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += to_f(h[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) bad |= !isfinite(acc[j]);
      store8(gsum + (i - v0) * 8, acc);
    }
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) {
    for (int q = 0; q < G; ++q) reinterpret_cast<uint32_t*>(flags.p[q])[found_base + my_rank] = 1u;
  }
  if (flag_b_base < 0) return;       // an intermediate bucket: the last launch of the step signals for all of them
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counter, 1u);
    if (done == gridDim.x - 1) {
      *counter = 0u;
      __threadfence_system();
      const uint32_t v = tag.value();
      for (int q = 0; q < G; ++q) st_release_sys(reinterpret_cast<uint32_t*>(flags.p[q]) + flag_b_base + my_rank, v);
    }
  }
}

// Ranges of 8-element vectors this rank updates: [v0, v1) of the flat buffer, whose reduced gradients start at
// vector g0 of gsum.  One range for the whole-buffer slice, one per bucket when the reduction was overlapped.
constexpr int kMaxRanges = 16;
struct VecRanges { int n; long long v0[kMaxRanges], v1[kMaxRanges], g0[kMaxRanges]; };

template <typename T>
__global__ void __launch_bounds__(256) adamw_shard_push_kernel(float* __restrict__ p32, float* __restrict__ m,
                                                               float* __restrict__ v, const float* __restrict__ gsum,
                                                               PeerPtrs p16, VecRanges rg, long long n_decay, int G, int my_rank,
                                                               const float* __restrict__ hp, float beta1, float beta2,
                                                               float eps, float wd, float grad_mult, PeerPtrs flags,
                                                               int flag_c_base, StepTag tag, unsigned* __restrict__ counter,
                                                               void* mc_p16) {
  if (hp[HP_FOUND_INF] == 0.f) {
    const float lr = hp[HP_LR_ENC];
    const float step = hp[HP_ADAM_STEP] + 1.0f;
    const float inv_scale = hp[HP_INV_SCALE] * grad_mult;
    const float inv_bc1 = 1.f / (1.f - powf(beta1, step)), inv_bc2 = 1.f / (1.f - powf(beta2, step));
    for (int ri = 0; ri < rg.n; ++ri) {
    const long long v0 = rg.v0[ri], v1 = rg.v1[ri], g0 = rg.g0[ri];
    for (long long i = v0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < v1; i += (long long)gridDim.x * blockDim.x) {
      const size_t e = (size_t)i * 8;
      float gg[8], pp[8], mm[8], vv[8];
      load8(gsum + (g0 + i - v0) * 8, gg);
      load8(p32 + e, pp);
      load8(m + e, mm);
      load8(v + e, vv);
      const float decay = ((long long)e < n_decay) ? 1.f - lr * wd : 1.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gr = gg[j] * inv_scale;
        mm[j] = beta1 * mm[j] + (1.f - beta1) * gr;
        vv[j] = beta2 * vv[j] + (1.f - beta2) * gr * gr;
        pp[j] = pp[j] * decay - lr * (mm[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + eps);
      }
      store8(p32 + e, pp);
      store8(m + e, mm);
      store8(v + e, vv);
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = from_f<T>(pp[j]);
      if (mc_p16 != nullptr) {
        multimem_st_v4(reinterpret_cast<T*>(mc_p16) + e, out);       // one store, every rank's copy
      } else {
        for (int q = 0; q < G; ++q) *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p16.p[q]) + e) = out;
      }
    }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counter, 1u);
    if (done == gridDim.x - 1) {
      *counter = 0u;
      __threadfence_system();
      const uint32_t t = tag.value();
      for (int q = 0; q < G; ++q) st_release_sys(reinterpret_cast<uint32_t*>(flags.p[q]) + flag_c_base + my_rank, t);
    }
  }
}

}  // namespace rb

using namespace rb;

static PeerPtrs make_ptrs(void* const* arr, int G) {
  PeerPtrs p{};
  for (int i = 0; i < G && i < kMaxPeers; ++i) p.p[i] = arr[i];
  return p;
}

RB_API int rb_step_inc(unsigned* step, cudaStream_t st) {
  step_inc_kernel<<<1, 32, 0, st>>>(step);
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_ag_push(const float* e, int b, int D, float p, const int* seed, unsigned stream_id, void* const* xbufs,
                      int row0, void* const* flags, int flag_base, int my_rank, int G, const unsigned* step_ptr,
                      unsigned* counters, cudaStream_t st) {
  if (G > kMaxPeers || (b * (long long)D) % 8) return -3;
  const long long n_vec = (long long)b * D / 8;
  int nblk = (int)((n_vec + 255) / 256);
  if (nblk > 16) nblk = 16;
  if (nblk < 1) nblk = 1;
  dim3 grid(G, nblk);
  ag_push_kernel<<<grid, 256, 0, st>>>(e, b, D, p, seed, stream_id, make_ptrs(xbufs, G), row0, make_ptrs(flags, G),
                                       flag_base, my_rank, StepTag{step_ptr, 1u, 0u}, counters);
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_peer_gather(const void* src, long long bytes, void* const* dst, long long slot_bytes, void* const* flags,
                          int flag_base, int my_rank, int G, const unsigned* step_ptr, unsigned* counters, cudaStream_t st) {
  if (G > kMaxPeers || bytes % 16 || slot_bytes % 16 || bytes < 16) return -3;
  const long long n16 = bytes / 16;
  int nblk = (int)((n16 + 255) / 256);
  if (nblk > 16) nblk = 16;
  dim3 grid(G, nblk);
  peer_gather_kernel<<<grid, 256, 0, st>>>((const uint4*)src, n16, make_ptrs(dst, G), slot_bytes / 16, make_ptrs(flags, G),
                                           flag_base, my_rank, StepTag{step_ptr, 1u, 0u}, counters);
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_rs_pull(void* const* partials, int G, int row0, int b, int D, float* de, const unsigned* my_flags,
                      const unsigned* step_ptr, float p, const int* seed, unsigned stream_id, int* status,
                      cudaStream_t st) {
  if (G > kMaxPeers || D % 4) return -3;
  rs_pull_kernel<<<b > 0 ? b : 1, 128, 0, st>>>(make_ptrs(partials, G), G, row0, b, D, de, my_flags,
                                                 StepTag{step_ptr, 1u, 0u}, p, seed, stream_id, status);
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_signal(void* const* flags, int G, int flag_base, int my_rank, const unsigned* step_ptr, unsigned mul,
                     unsigned add, cudaStream_t st) {
  if (G > kMaxPeers) return -3;
  signal_kernel<<<1, 32, 0, st>>>(make_ptrs(flags, G), G, flag_base, my_rank, StepTag{step_ptr, mul, add});
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_wait_flags(const unsigned* my_flags, int G, const unsigned* step_ptr, unsigned mul, unsigned add,
                         unsigned* found_words, float* hp, int* status, cudaStream_t st) {
  if (G > kMaxPeers) return -3;
  wait_flags_kernel<<<1, 32, 0, st>>>(my_flags, G, StepTag{step_ptr, mul, add}, found_words, hp, status);
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_grad_allreduce(int dtype, void* const* grads, long long lo, long long hi, int G, int my_rank,
                             const unsigned* my_flags_a, void* const* flags, int flag_b_base, int found_base,
                             const unsigned* step_ptr, unsigned mul, unsigned add, unsigned* counter, int blocks,
                             int* status, cudaStream_t st) {
  if (G > kMaxPeers || lo % 8 || hi % 8 || hi < lo) return -3;
  if (blocks < 1) blocks = 1;
  PeerPtrs g = make_ptrs(grads, G), f = make_ptrs(flags, G);
  const StepTag tag{step_ptr, mul, add};
  switch (dtype) {
    case RB_BF16:
      grad_allreduce_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(g, lo, hi, G, my_rank, my_flags_a, tag, f, flag_b_base,
                                                                   found_base, tag, counter, status);
      break;
    case RB_F16:
      grad_allreduce_kernel<__half><<<blocks, 256, 0, st>>>(g, lo, hi, G, my_rank, my_flags_a, tag, f, flag_b_base,
                                                            found_base, tag, counter, status);
      break;
    default:
      return -1;  // fp32 encoders use the library all-reduce
  }
  RB_LAUNCH_CHECK();
  return 0;
}

// Reduce-scatter of vectors [v0, v1) (8 elements each) of the flat gradient buffer into gsum[0 .. (v1-v0)*8): the
// sums over all ranks.  Waits until every rank's progress flag (class A) has reached step * mul_a + add_a; with
// flag_b_base >= 0 raises "reduced" (class B, value step) on every rank afterwards.
RB_API int rb_grad_reduce_scatter_range(int dtype, void* const* grads, long long v0, long long v1, int G, int my_rank,
                                        const unsigned* my_flags_a, const unsigned* step_ptr, unsigned mul_a, unsigned add_a,
                                        float* gsum, void* const* flags, int flag_b_base, int found_base, unsigned* counter,
                                        int blocks, int* status, const void* mc_grads, cudaStream_t st) {
  if (G > kMaxPeers || v0 < 0 || v1 < v0) return -3;
  if (blocks < 1) blocks = 1;
  PeerPtrs g = make_ptrs(grads, G), f = make_ptrs(flags, G);
  const StepTag tag_a{step_ptr, mul_a, add_a}, tag{step_ptr, 1u, 0u};
  if (dtype == RB_BF16)
    grad_reduce_scatter_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(g, v0, v1, G, my_rank, my_flags_a, tag_a, tag, gsum, f, flag_b_base, found_base, counter, status, mc_grads);
  else if (dtype == RB_F16)
    grad_reduce_scatter_kernel<__half><<<blocks, 256, 0, st>>>(g, v0, v1, G, my_rank, my_flags_a, tag_a, tag, gsum, f, flag_b_base, found_base, counter, status, mc_grads);
  else
    return -1;
  RB_LAUNCH_CHECK();
  return 0;
}

// This rank's contiguous 1/G slice of the whole buffer (n elements), progress tag = step.
RB_API int rb_grad_reduce_scatter(int dtype, void* const* grads, long long n, int G, int my_rank,
                                  const unsigned* my_flags_a, const unsigned* step_ptr, float* gsum, void* const* flags,
                                  int flag_b_base, int found_base, unsigned* counter, int blocks, int* status,
                                  const void* mc_grads, cudaStream_t st) {
  if (n % 8) return -3;
  const long long n_vec = n / 8, per = (n_vec + G - 1) / G;
  const long long v0 = per * my_rank < n_vec ? per * my_rank : n_vec;
  const long long v1 = per * (my_rank + 1) < n_vec ? per * (my_rank + 1) : n_vec;
  return rb_grad_reduce_scatter_range(dtype, grads, v0, v1, G, my_rank, my_flags_a, step_ptr, 1u, 0u, gsum, flags,
                                      flag_b_base, found_base, counter, blocks, status, mc_grads, st);
}

// AdamW on the vector ranges [v0[i], v1[i]) whose reduced gradients start at vector g0[i] of gsum, then the push of
// the updated 16-bit values into every rank's compute copy and the "pushed" flag (class C).
RB_API int rb_adamw_ranges_push(int dtype, float* p32, float* m, float* v, const float* gsum, void* const* p16,
                                int n_ranges, const long long* v0, const long long* v1, const long long* g0,
                                long long n_decay, int G, int my_rank, const float* hp, float beta1, float beta2, float eps,
                                float wd, float grad_mult, void* const* flags, int flag_c_base, const unsigned* step_ptr,
                                unsigned* counter, int blocks, void* mc_p16, cudaStream_t st) {
  if (G > kMaxPeers || n_decay % 8 || n_ranges < 0 || n_ranges > kMaxRanges) return -3;
  if (blocks < 1) blocks = 1;
  VecRanges rg{};
  rg.n = n_ranges;
  for (int i = 0; i < n_ranges; ++i) { rg.v0[i] = v0[i]; rg.v1[i] = v1[i]; rg.g0[i] = g0[i]; }
  PeerPtrs pp = make_ptrs(p16, G), f = make_ptrs(flags, G);
  const StepTag tag{step_ptr, 1u, 0u};
  if (dtype == RB_BF16)
    adamw_shard_push_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(p32, m, v, gsum, pp, rg, n_decay, G, my_rank, hp, beta1, beta2, eps, wd, grad_mult, f, flag_c_base, tag, counter, mc_p16);
  else if (dtype == RB_F16)
    adamw_shard_push_kernel<__half><<<blocks, 256, 0, st>>>(p32, m, v, gsum, pp, rg, n_decay, G, my_rank, hp, beta1, beta2, eps, wd, grad_mult, f, flag_c_base, tag, counter, mc_p16);
  else
    return -1;
  RB_LAUNCH_CHECK();
  return 0;
}

RB_API int rb_adamw_shard_push(int dtype, float* p32, float* m, float* v, const float* gsum, void* const* p16,
                               long long n, long long n_decay, int G, int my_rank, const float* hp, float beta1,
                               float beta2, float eps, float wd, float grad_mult, void* const* flags, int flag_c_base,
                               const unsigned* step_ptr, unsigned* counter, int blocks, void* mc_p16, cudaStream_t st) {
  if (n % 8) return -3;
  const long long n_vec = n / 8, per = (n_vec + G - 1) / G;
  const long long v0 = per * my_rank < n_vec ? per * my_rank : n_vec;
  const long long v1 = per * (my_rank + 1) < n_vec ? per * (my_rank + 1) : n_vec;
  const long long g0 = 0;
  return rb_adamw_ranges_push(dtype, p32, m, v, gsum, p16, 1, &v0, &v1, &g0, n_decay, G, my_rank, hp, beta1, beta2, eps, wd,
                              grad_mult, flags, flag_c_base, step_ptr, counter, blocks, mc_p16, st);
}

// ------------------------------------------------------------------------------------ peer-mapped allocations
// Plain CUDA IPC: a cudaMalloc'd buffer is exported with cudaIpcGetMemHandle and mapped by the other ranks'
// processes with cudaIpcOpenMemHandle.  Such a mapping is peer-to-peer only -- it never binds an NVLink
// multicast object -- which is what the default (NVLS off) configuration wants: a rank that dies while
// its memory is bound to a multicast object can fault the surviving ranks' GPUs.
RB_API int rb_ipc_alloc(long long bytes, void** out) {
  if (bytes < 1 || out == nullptr) return -3;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) { cudaFree(p); return (int)e; }
  *out = p;
  return 0;
}
RB_API int rb_ipc_free(void* p) { return (int)cudaFree(p); }
RB_API int rb_ipc_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }
RB_API int rb_ipc_export(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
RB_API int rb_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
RB_API int rb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
