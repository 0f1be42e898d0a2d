// Optimizer steps fused with the gradient collective over NVLink peer memory.
//
// The gradient of every element is the average of the copies that the W ranks
// hold in a symmetric buffer (same layout at the same offset on every GPU,
// each mapped into every process).  One kernel per rank reads the W copies
// straight into registers -- plain peer loads in a fixed rank order, or one
// multimem.ld_reduce through the NVSwitch when a multicast mapping exists --
// and runs the same per-unit update as the local step kernels, so the reduced
// gradient never exists in HBM and no collective library is involved:
//   * DDP bucket: every rank reduces the whole bucket and updates its replica
//     (one-shot all-reduce fused with the update; rank order is fixed, so all
//     replicas compute bit-identical sums);
//   * FSDP2: rank r reduces only row r of the [W, shard] reduce-scatter input
//     and updates its shard (reduce-scatter fused with the sharded update).
// The reference leaves both collectives to NCCL inside PyTorch's DDP / FSDP2
// and then launches its update per tensor (flashoptim/optimizers.py:597-616).
//
// Cross-GPU ordering uses epoch flags in a symmetric "signal pad": word
// [channel * FO_MAX_PEERS + src] of rank d's pad is written only by rank src.
// Every wait is bounded by a wall-clock limit (globaltimer); a wait that runs
// out records a code in a local status word, the kernel skips its work and
// returns normally, and the host raises.  No TMA or multicast-cluster loads
// are used anywhere in this file.
#include "fo_step_core.cuh"

namespace fo {

constexpr int kCommThreads = 256;
constexpr int kCommChunk = kCommThreads * kUnit;
constexpr int kCommCtasPerSm = 3;

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Epochs only grow; a flag satisfies a wait once it has reached the epoch
// (signed difference, so wrap-around after 2^31 steps is harmless).
__device__ __forceinline__ bool epoch_reached(uint32_t flag, uint32_t epoch) {
  return (int32_t)(flag - epoch) >= 0;
}

// Thread `t < world` waits until rank t's flag on `channel` reaches `epoch`.
// Returns false on timeout (and records it).
__device__ __forceinline__ bool wait_flag(const FoCommArgs& A, int channel, int src, uint32_t epoch) {
  const uint32_t* flag = A.pad[A.rank] + channel * FO_MAX_PEERS + src;
  const uint64_t t0 = global_ns();
  for (;;) {
    if (epoch_reached(ld_acquire_sys(flag), epoch)) return true;
    if (global_ns() - t0 > A.timeout_ns) {
      atomicOr(reinterpret_cast<unsigned int*>(A.status), 1u << (channel & 31));
      atomicExch(reinterpret_cast<unsigned int*>(A.status) + 1, (unsigned int)src + 1u);
      return false;
    }
    __nanosleep(64);
  }
}

// Every CTA: wait until all ranks have published `epoch` on the ready channel.
// CTA 0 also publishes this rank's own arrival first.  Returns false (for the
// whole CTA) if any wait ran out.
__device__ __forceinline__ bool start_barrier(const FoCommArgs& A) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < A.world) {
    __threadfence_system();
    st_release_sys(A.pad[threadIdx.x] + A.ready_channel * FO_MAX_PEERS + A.rank, A.epoch);
  }
  if (threadIdx.x < A.world) {
    if (!wait_flag(A, A.ready_channel, threadIdx.x, A.epoch)) ok = 0;
  }
  __syncthreads();
  return ok != 0;
}

// After the main loop: the last CTA to finish tells every peer that this rank
// no longer reads their buffers for `epoch` (done channel).
// `counter` selects the status word that counts finished CTAs: kernels that may run at the
// same time on one GPU (a step kernel on the reduce-scatter stream and an all-gather on the
// all-gather stream) must not share one.
// `remote_stores`: the kernel wrote into other ranks' memory; every CTA then orders its stores
// at system scope before it counts itself as finished.
__device__ __forceinline__ void end_signal(const FoCommArgs& A, int counter = 2, bool remote_stores = false) {
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (remote_stores || A.push) __threadfence_system();  // this CTA's stores into the peers' memory
    else __threadfence();
    unsigned int n = atomicAdd(reinterpret_cast<unsigned int*>(A.status) + counter, 1u);
    last = (n == gridDim.x - 1);
    if (last) reinterpret_cast<unsigned int*>(A.status)[counter] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (last && threadIdx.x < A.world) {
    __threadfence_system();
    st_release_sys(A.pad[threadIdx.x] + A.done_channel * FO_MAX_PEERS + A.rank, A.epoch);
    if (A.push) st_release_sys(A.pad[threadIdx.x] + A.pushed_channel * FO_MAX_PEERS + A.rank, A.push_epoch);
  }
}

// ---------------------------------------------------------------- gradient from peers

__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f32x4(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__device__ __forceinline__ void multimem_st16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Remote part of one unit: the W copies (peer loads) or the switch-reduced copy
// (multimem) are requested here and only consumed by peer_sum(), so a thread can
// have the loads of several units in flight.  `off` is the byte offset of the
// unit inside every rank's buffer; kPeers bounds the world size at compile time.
template <typename T, int kPeers>
__device__ __forceinline__ void peer_load(const FoCommArgs& A, int64_t off, int cnt, bool vec,
                                          Raw8<T> (&r)[kPeers]) {
  if (cnt <= 0) return;
  if (vec && A.multicast != nullptr) {
    const char* a = static_cast<const char*>(A.multicast) + off;
    if constexpr (sizeof(T) == 4) {
      r[0].v = multimem_ld_reduce_f32x4(a);
      r[0].w = multimem_ld_reduce_f32x4(a + 16);
    } else if constexpr (Elem<T>::kMant == 7) {
      r[0].v = multimem_ld_reduce_bf16x8(a);
    } else {
      r[0].v = multimem_ld_reduce_f16x8(a);
    }
    return;
  }
#pragma unroll
  for (int p = 0; p < kPeers; ++p) {
    if (p < A.world) {
      const T* src = reinterpret_cast<const T*>(static_cast<const char*>(A.grad[p]) + off);
      r[p].v = make_uint4(0, 0, 0, 0);
      if constexpr (sizeof(T) == 4) r[p].w = make_uint4(0, 0, 0, 0);
      if (vec) load_raw8<T>(r[p], src, true);
      else load_raw8_partial<T>(r[p], src, cnt);
    }
  }
}
// Sum in fp32, in rank order (every replica adds in the same order).
template <typename T, int kPeers>
__device__ __forceinline__ void peer_sum(const FoCommArgs& A, int cnt, bool vec, const Raw8<T> (&r)[kPeers],
                                         float2 (&g)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) g[i] = make_float2(0.f, 0.f);
  if (cnt <= 0) return;
  if (vec && A.multicast != nullptr) {
    unpack8<T>(r[0], g);
    return;
  }
#pragma unroll
  for (int p = 0; p < kPeers; ++p) {
    if (p < A.world) {
      float2 x[4];
      unpack8<T>(r[p], x);
#pragma unroll
      for (int i = 0; i < 4; ++i) g[i] = add2(g[i], x[i]);
    }
  }
}
template <typename T>
__device__ __forceinline__ void reduce_unit(const FoCommArgs& A, int64_t off, int cnt, bool vec,
                                            float2 (&g)[4]) {
  Raw8<T> r[FO_MAX_PEERS];
  peer_load<T, FO_MAX_PEERS>(A, off, cnt, vec, r);
  peer_sum<T, FO_MAX_PEERS>(A, cnt, vec, r, g);
}

struct CommWalker {
  const FoSeg* segs;
  const int32_t* cb;
  int seg, seg_begin, seg_end;
  FoSeg S;
  bool vec;
  __device__ __forceinline__ CommWalker(const FoSeg* s, const int32_t* c) : segs(s), cb(c), seg(0) {
    seg_begin = cb[0];
    seg_end = cb[1];
    S = segs[0];
    vec = vector_safe();
  }
  // S.g holds a byte offset into the symmetric buffers here, not a pointer
  __device__ __forceinline__ bool vector_safe() const {
    uintptr_t a = reinterpret_cast<uintptr_t>(S.p) | reinterpret_cast<uintptr_t>(S.g) |
                  reinterpret_cast<uintptr_t>(S.ecc) | reinterpret_cast<uintptr_t>(S.s0) |
                  reinterpret_cast<uintptr_t>(S.s1);
    return (a & 15) == 0;
  }
  __device__ __forceinline__ void seek(int c) {
    if (c >= seg_end) {
      do { ++seg; } while (c >= cb[seg + 1]);
      S = segs[seg];
      seg_begin = cb[seg];
      seg_end = cb[seg + 1];
      vec = vector_safe();
    }
  }
};

// Writes the averaged gradient of one unit to `grad_out` (optional).
template <typename T>
__device__ __forceinline__ void store_grad_out(const FoCommArgs& A, int64_t goff, int cnt, bool vec,
                                               const float2 (&g)[4], float scale) {
  if (A.grad_out == nullptr || cnt <= 0) return;
  float2 s[4], back[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = mul2(g[i], splat2(scale));
  Raw8<T> r;
  pack8<T>(s, r, back);
  T* dst = reinterpret_cast<T*>(static_cast<char*>(A.grad_out) + (goff - A.grad_out_sub));
  const bool v = vec && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
  store_raw8<T>(r, dst, cnt, v);
}

// All-gather on write: the freshly narrowed parameter unit goes to the same offset of
// every rank's parameter buffer (W peer stores, or one multimem.st replicated by the switch).
template <typename T, int kPeers>
__device__ __forceinline__ void push_param(const FoCommArgs& A, int64_t off, int cnt, bool vec,
                                           const Raw8<T>& pn) {
  if (cnt <= 0) return;
  off += A.param_out_delta;
  if (vec && A.param_out_mc != nullptr && (off & 15) == 0) {
    char* d = static_cast<char*>(A.param_out_mc) + off;
    multimem_st16(d, pn.v);
    if constexpr (sizeof(T) == 4) multimem_st16(d + 16, pn.w);
    return;
  }
#pragma unroll
  for (int p = 0; p < kPeers; ++p) {
    if (p < A.world) {
      T* d = reinterpret_cast<T*>(static_cast<char*>(A.param_out[p]) + off);
      const bool v = vec && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
      store_raw8<T>(pn, d, cnt, v);
    }
  }
}

// Units per thread by world size: the fewer ranks, the fewer remote loads one unit
// issues, so more units are put in flight per thread (2 ranks: 4 units, 3-4 ranks: 2,
// 5-8 ranks: 1); remote requests in flight per thread stay at 8 x 16 bytes.
template <int kU>
struct PeerCfg {
  static constexpr int kPeers = FO_MAX_PEERS / kU;
  static constexpr int kChunk = kCommThreads * kUnit * kU;
  static constexpr int kCtas = kU == 1 ? kCommCtasPerSm : 2;
};

template <typename T, int kErr, int kStates, bool kQ, int kU, typename Hyper, typename Update>
__device__ __forceinline__ void peer_step_body(const FoSeg* segs, const int32_t* cb, int total_chunks,
                                               const Hyper& H, const FoCommArgs& A, Update update) {
  using Regs = UnitRegs<T, kErr, kStates, kQ>;
  constexpr int kPeers = PeerCfg<kU>::kPeers;
  CommWalker w(segs, cb);
  for (int c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    w.seek(c);
    const int64_t chunk_base = (int64_t)(c - w.seg_begin) * PeerCfg<kU>::kChunk;
    const int64_t g0 = (int64_t)reinterpret_cast<intptr_t>(w.S.g);
    Raw8<T> remote[kU][kPeers];
    int cnt[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t base = chunk_base + (int64_t)(u * kCommThreads + threadIdx.x) * kUnit;
      const int64_t left = w.S.n - base;
      cnt[u] = left >= kUnit ? kUnit : (int)left;
      peer_load<T, kPeers>(A, g0 + base * (int64_t)sizeof(T), cnt[u], w.vec && cnt[u] == kUnit, remote[u]);
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t base = chunk_base + (int64_t)(u * kCommThreads + threadIdx.x) * kUnit;
      Regs r;
      load_unit_state(r, w.S, base, w.vec);
      const bool vec = w.vec && r.cnt == kUnit;
      float2 p[4], g[4], m[4], v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) m[i] = v[i] = make_float2(0.f, 0.f);
      peer_sum<T, kPeers>(A, r.cnt, vec, remote[u], g);
      store_grad_out<T>(A, g0 + base * (int64_t)sizeof(T), r.cnt, vec, g, H.grad_scale);
      widen_unit(r, p, m, v);
      update(p, g, m, v, H);
      Raw8<T> pn;
      store_unit(r, w.S, base, w.vec, p, m, v, pn);
      if (A.push) push_param<T, kPeers>(A, g0 + base * (int64_t)sizeof(T), r.cnt, vec, pn);
    }
  }
}

template <bool kQ>
struct PeerAdamUpdate {
  __device__ __forceinline__ void operator()(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4], float2 (&v)[4],
                                             const FoAdamHyper& H) const {
    adam_update8<kQ>(p, g, m, v, H);
  }
};
template <bool kHasState>
struct PeerMomentumUpdate {
  __device__ __forceinline__ void operator()(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4], float2 (&v)[4],
                                             const FoMomentumHyper& H) const {
    momentum_update8(p, g, m, H, kHasState);
  }
};

template <typename T, int kErr, bool kQ, int kU>
__global__ void __launch_bounds__(kCommThreads, PeerCfg<kU>::kCtas)
    adam_peer_kernel(const FoSeg* __restrict__ segs, const int32_t* __restrict__ cb, int total_chunks,
                     const __grid_constant__ FoAdamHyper H, const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) return;
  peer_step_body<T, kErr, 2, kQ, kU>(segs, cb, total_chunks, H, A, PeerAdamUpdate<kQ>());
  end_signal(A);
}

template <typename T, int kErr, int kMode, int kU>
__global__ void __launch_bounds__(kCommThreads, PeerCfg<kU>::kCtas)
    momentum_peer_kernel(const FoSeg* __restrict__ segs, const int32_t* __restrict__ cb, int total_chunks,
                         const __grid_constant__ FoMomentumHyper H, const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) return;
  constexpr int kStates = kMode == FO_STATE_NONE ? 0 : 1;
  constexpr bool kQ = kMode == FO_STATE_Q8;
  peer_step_body<T, kErr, kStates, kQ, kU>(segs, cb, total_chunks, H, A, PeerMomentumUpdate<(kStates > 0)>());
  end_signal(A);
}

// Plain averaged reduce (no update): out[i] = scale * sum_r peer_r[off + i].
// DDP buckets that must hand reduced gradients back, and the baseline for the
// fused kernels' comparisons.
template <typename T>
__global__ void __launch_bounds__(kCommThreads, kCommCtasPerSm)
    reduce_peer_kernel(int64_t n, int64_t src_off, T* __restrict__ out, float scale,
                       const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) return;
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  const bool aligned = ((src_off | reinterpret_cast<intptr_t>(out)) & 15) == 0;
  for (int64_t u = (int64_t)blockIdx.x * kCommThreads + threadIdx.x; u < n_units;
       u += (int64_t)gridDim.x * kCommThreads) {
    const int64_t base = u * kUnit;
    const int64_t left = n - base;
    const int cnt = left >= kUnit ? kUnit : (int)left;
    const bool vec = aligned && cnt == kUnit;
    float2 g[4], s[4], back[4];
    reduce_unit<T>(A, src_off + base * (int64_t)sizeof(T), cnt, vec, g);
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = mul2(g[i], splat2(scale));
    Raw8<T> r;
    pack8<T>(s, r, back);
    store_raw8<T>(r, out + base, cnt, vec);
  }
  end_signal(A);
}

// Two-shot all-reduce, first shot: rank r averages slice r of the n elements at
// `src_off` of every rank's buffer and stores the result into the same slice at
// `dst_off` of EVERY rank's buffer (peer stores, or one multimem.st through the
// switch).  After all ranks published done(epoch) each buffer holds the complete
// averaged vector at `dst_off`; a local step kernel then reads it from its own HBM.
template <typename T>
__global__ void __launch_bounds__(kCommThreads, kCommCtasPerSm)
    reduce_bcast_peer_kernel(int64_t n, int64_t src_off, int64_t dst_off, float scale,
                             const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) return;
  // slices are multiples of 8 elements so that every unit of a slice is whole
  const int64_t slice = ((n + (int64_t)A.world * kUnit - 1) / ((int64_t)A.world * kUnit)) * kUnit;
  const int64_t begin = slice * A.rank;
  const int64_t end = begin + slice < n ? begin + slice : n;
  const int64_t n_units = end > begin ? (end - begin + kUnit - 1) / kUnit : 0;
  const bool aligned = ((src_off | dst_off) & 15) == 0;
  for (int64_t u = (int64_t)blockIdx.x * kCommThreads + threadIdx.x; u < n_units;
       u += (int64_t)gridDim.x * kCommThreads) {
    const int64_t base = begin + u * kUnit;
    const int64_t left = end - base;
    const int cnt = left >= kUnit ? kUnit : (int)left;
    const bool vec = aligned && cnt == kUnit;
    float2 g[4], s[4], back[4];
    reduce_unit<T>(A, src_off + base * (int64_t)sizeof(T), cnt, vec, g);
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = mul2(g[i], splat2(scale));
    Raw8<T> r;
    pack8<T>(s, r, back);
    const int64_t off = dst_off + base * (int64_t)sizeof(T);
    if (vec && A.multicast != nullptr) {
      char* d = static_cast<char*>(const_cast<void*>(A.multicast)) + off;
      multimem_st16(d, r.v);
      if constexpr (sizeof(T) == 4) multimem_st16(d + 16, r.w);
    } else {
      for (int p = 0; p < A.world; ++p) {
        T* d = reinterpret_cast<T*>(static_cast<char*>(const_cast<void*>(A.grad[p])) + off);
        store_raw8<T>(r, d, cnt, vec);
      }
    }
  }
  end_signal(A, 2, true);
}

// All-gather by pulling: rank r copies slot s of rank s's buffer (at s * slot_bytes)
// into slot s of its own buffer, for every s != r.  Buffers are symmetric.
__global__ void __launch_bounds__(kCommThreads, kCommCtasPerSm)
    allgather_pull_kernel(int64_t slot_bytes, const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) return;
  const int64_t n16 = slot_bytes / 16;  // slots are multiples of 16 bytes (checked by the host)
  for (int s = 0; s < A.world; ++s) {
    if (s == A.rank) continue;
    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const char*>(A.grad[s]) + s * slot_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(const_cast<void*>(A.grad[A.rank])) + s * slot_bytes);
    for (int64_t i = (int64_t)blockIdx.x * kCommThreads + threadIdx.x; i < n16;
         i += (int64_t)gridDim.x * kCommThreads)
      dst[i] = src[i];
  }
  end_signal(A, 3);
}

// Stand-alone flag operations (one CTA).
__global__ void signal_kernel(const __grid_constant__ FoCommArgs A, int channel) {
  if (threadIdx.x < A.world) {
    __threadfence_system();
    st_release_sys(A.pad[threadIdx.x] + channel * FO_MAX_PEERS + A.rank, A.epoch);
  }
}
__global__ void wait_kernel(const __grid_constant__ FoCommArgs A, int channel) {
  if (threadIdx.x < A.world) wait_flag(A, channel, threadIdx.x, A.epoch);
}

static int units_for_world(int world) { return world <= 2 ? 4 : (world <= 4 ? 2 : 1); }

static int comm_grid(int64_t work_ctas, const FoCommArgs* a, int ctas_per_sm = kCommCtasPerSm) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  int64_t g = (int64_t)sms * ctas_per_sm;
  if (a && a->max_ctas > 0 && a->max_ctas < g) g = a->max_ctas;
  if (work_ctas < g) g = work_ctas;
  return g < 1 ? 1 : (int)g;
}

static bool args_ok(const FoCommArgs* a) {
  return a && a->world >= 1 && a->world <= FO_MAX_PEERS && a->rank >= 0 && a->rank < a->world && a->status;
}

template <typename T, int kErr, int kU>
static int launch_adam_peer_q(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                              const FoCommArgs& A, int quantized, cudaStream_t st) {
  const int grid = comm_grid(total, &A, PeerCfg<kU>::kCtas);
  if (quantized) adam_peer_kernel<T, kErr, true, kU><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
  else adam_peer_kernel<T, kErr, false, kU><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
  return (int)cudaGetLastError();
}
template <typename T, int kErr>
static int launch_adam_peer_u(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                              const FoCommArgs& A, int quantized, cudaStream_t st) {
  switch (units_for_world(A.world)) {
    case 4: return launch_adam_peer_q<T, kErr, 4>(s, cb, total, H, A, quantized, st);
    case 2: return launch_adam_peer_q<T, kErr, 2>(s, cb, total, H, A, quantized, st);
  }
  return launch_adam_peer_q<T, kErr, 1>(s, cb, total, H, A, quantized, st);
}
template <typename T>
static int launch_adam_peer(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                            const FoCommArgs& A, int err, int quantized, cudaStream_t st) {
  if constexpr (Elem<T>::kNarrow) {
    if (err == 1) return launch_adam_peer_u<T, 1>(s, cb, total, H, A, quantized, st);
    if (err == 2) return launch_adam_peer_u<T, 2>(s, cb, total, H, A, quantized, st);
  }
  if (err != 0) return (int)cudaErrorInvalidValue;
  return launch_adam_peer_u<T, 0>(s, cb, total, H, A, quantized, st);
}

template <typename T, int kErr, int kU>
static int launch_mom_peer_m(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                             const FoCommArgs& A, int mode, cudaStream_t st) {
  const int grid = comm_grid(total, &A, PeerCfg<kU>::kCtas);
  switch (mode) {
    case FO_STATE_NONE:
      momentum_peer_kernel<T, kErr, FO_STATE_NONE, kU><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
      break;
    case FO_STATE_Q8:
      momentum_peer_kernel<T, kErr, FO_STATE_Q8, kU><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
      break;
    case FO_STATE_FULL:
      momentum_peer_kernel<T, kErr, FO_STATE_FULL, kU><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
      break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}
template <typename T, int kErr>
static int launch_mom_peer_u(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                             const FoCommArgs& A, int mode, cudaStream_t st) {
  switch (units_for_world(A.world)) {
    case 4: return launch_mom_peer_m<T, kErr, 4>(s, cb, total, H, A, mode, st);
    case 2: return launch_mom_peer_m<T, kErr, 2>(s, cb, total, H, A, mode, st);
  }
  return launch_mom_peer_m<T, kErr, 1>(s, cb, total, H, A, mode, st);
}
template <typename T>
static int launch_mom_peer(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                           const FoCommArgs& A, int err, int mode, cudaStream_t st) {
  if constexpr (Elem<T>::kNarrow) {
    if (err == 1) return launch_mom_peer_u<T, 1>(s, cb, total, H, A, mode, st);
    if (err == 2) return launch_mom_peer_u<T, 2>(s, cb, total, H, A, mode, st);
  }
  if (err != 0) return (int)cudaErrorInvalidValue;
  return launch_mom_peer_u<T, 0>(s, cb, total, H, A, mode, st);
}

}  // namespace fo

extern "C" int fo_comm_chunk_elems(int world) { return fo::kCommChunk * fo::units_for_world(world); }

extern "C" int fo_adam_step_peer(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                                 int dtype, int err_bytes, int quantized, const FoAdamHyper* hyper,
                                 const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm) || !hyper) return (int)cudaErrorInvalidValue;
  if (n_seg <= 0 || total_chunks <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FO_BF16:
      return fo::launch_adam_peer<__nv_bfloat16>(segs, chunk_begin, total_chunks, *hyper, *comm, err_bytes,
                                                 quantized, st);
    case FO_FP16:
      return fo::launch_adam_peer<__half>(segs, chunk_begin, total_chunks, *hyper, *comm, err_bytes, quantized, st);
    case FO_FP32:
      return fo::launch_adam_peer<float>(segs, chunk_begin, total_chunks, *hyper, *comm, err_bytes, quantized, st);
  }
  return (int)cudaErrorInvalidValue;
}

extern "C" int fo_momentum_step_peer(const FoSeg* segs, const int32_t* chunk_begin, int n_seg,
                                     int total_chunks, int dtype, int err_bytes, int state_mode,
                                     const FoMomentumHyper* hyper, const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm) || !hyper) return (int)cudaErrorInvalidValue;
  if (n_seg <= 0 || total_chunks <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FO_BF16:
      return fo::launch_mom_peer<__nv_bfloat16>(segs, chunk_begin, total_chunks, *hyper, *comm, err_bytes,
                                                state_mode, st);
    case FO_FP16:
      return fo::launch_mom_peer<__half>(segs, chunk_begin, total_chunks, *hyper, *comm, err_bytes, state_mode, st);
    case FO_FP32:
      return fo::launch_mom_peer<float>(segs, chunk_begin, total_chunks, *hyper, *comm, err_bytes, state_mode, st);
  }
  return (int)cudaErrorInvalidValue;
}

extern "C" int fo_reduce_peer(int64_t n, int64_t src_offset_bytes, void* out, int dtype, float scale,
                              const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm)) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  const int grid = fo::comm_grid((n + fo::kCommChunk - 1) / fo::kCommChunk, comm);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FO_BF16:
      fo::reduce_peer_kernel<<<grid, fo::kCommThreads, 0, st>>>(n, src_offset_bytes, (__nv_bfloat16*)out, scale,
                                                                *comm);
      break;
    case FO_FP16:
      fo::reduce_peer_kernel<<<grid, fo::kCommThreads, 0, st>>>(n, src_offset_bytes, (__half*)out, scale, *comm);
      break;
    case FO_FP32:
      fo::reduce_peer_kernel<<<grid, fo::kCommThreads, 0, st>>>(n, src_offset_bytes, (float*)out, scale, *comm);
      break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int fo_reduce_bcast_peer(int64_t n, int64_t src_offset_bytes, int64_t dst_offset_bytes, int dtype,
                                    float scale, const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm)) return (int)cudaErrorInvalidValue;
  if (n <= 0) return 0;
  const int64_t per_rank = (n + comm->world - 1) / comm->world;
  const int grid = fo::comm_grid((per_rank + fo::kCommChunk - 1) / fo::kCommChunk, comm);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FO_BF16:
      fo::reduce_bcast_peer_kernel<__nv_bfloat16><<<grid, fo::kCommThreads, 0, st>>>(n, src_offset_bytes,
                                                                                      dst_offset_bytes, scale, *comm);
      break;
    case FO_FP16:
      fo::reduce_bcast_peer_kernel<__half><<<grid, fo::kCommThreads, 0, st>>>(n, src_offset_bytes, dst_offset_bytes,
                                                                               scale, *comm);
      break;
    case FO_FP32:
      fo::reduce_bcast_peer_kernel<float><<<grid, fo::kCommThreads, 0, st>>>(n, src_offset_bytes, dst_offset_bytes,
                                                                              scale, *comm);
      break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int fo_allgather_peer(int64_t slot_bytes, const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm) || slot_bytes < 0 || (slot_bytes & 15)) return (int)cudaErrorInvalidValue;
  if (slot_bytes == 0) return 0;
  const int grid = fo::comm_grid((slot_bytes / 16 + fo::kCommThreads - 1) / fo::kCommThreads, comm);
  fo::allgather_pull_kernel<<<grid, fo::kCommThreads, 0, static_cast<cudaStream_t>(stream)>>>(slot_bytes, *comm);
  return (int)cudaGetLastError();
}

extern "C" int fo_comm_signal(const FoCommArgs* comm, int channel, void* stream) {
  if (!fo::args_ok(comm)) return (int)cudaErrorInvalidValue;
  fo::signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(*comm, channel);
  return (int)cudaGetLastError();
}

extern "C" int fo_comm_wait(const FoCommArgs* comm, int channel, void* stream) {
  if (!fo::args_ok(comm)) return (int)cudaErrorInvalidValue;
  fo::wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(*comm, channel);
  return (int)cudaGetLastError();
}
