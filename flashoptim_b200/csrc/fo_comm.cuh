// Device helpers shared by the kernels that fuse a gradient collective with the update.  No
// counterpart in the reference, which leaves every collective to DDP / FSDP2 and NCCL and steps
// afterwards (gradient-release hook: flashoptim/optimizers.py:3019-3051).
//
// Used by fo_comm.cu (register path) and fo_comm_staged.cu (bulk-copy staged path): epoch flags with
// bounded waits, the start barrier / end signal of a kernel, multimem instructions, the
// walker over a segment table whose gradient entries are byte offsets into symmetric
// buffers, and the stores that hand the averaged gradient back and push the new parameters.
#pragma once

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
  if (A.flags & FO_COMM_NO_BARRIER) return true;  // the caller synchronised the ranks itself
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
// `completed` is false for a CTA whose start barrier ran out: it still counts itself (so the
// counter is back at zero when the kernel ends, whatever mixture of CTAs timed out) but never
// publishes anything.
__device__ __forceinline__ void end_signal(const FoCommArgs& A, int counter = 2, bool remote_stores = false,
                                           bool completed = true) {
  if (A.flags & FO_COMM_NO_SIGNAL) return;  // the caller publishes the flags itself
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (remote_stores || A.push) __threadfence_system();  // this CTA's stores into the peers' memory
    else __threadfence();
    unsigned int n = atomicAdd(reinterpret_cast<unsigned int*>(A.status) + counter, 1u);
    last = (n == gridDim.x - 1);
    if (last) atomicExch(reinterpret_cast<unsigned int*>(A.status) + counter, 0u);  // ready for the next launch
  }
  __syncthreads();
  if (completed && last && threadIdx.x < A.world) {
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
  if (A.flags & FO_COMM_PUSH_LOCAL) {
    T* d = reinterpret_cast<T*>(static_cast<char*>(A.param_out[A.rank]) + off);
    store_raw8<T>(pn, d, cnt, vec && ((reinterpret_cast<uintptr_t>(d) & 15) == 0));
    return;
  }
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

// Slow path of one unit (tail of a tensor, or a tensor whose addresses are not 16-byte
// aligned): element-wise peer loads, summed at once in rank order.
template <typename T>
__device__ __noinline__ void reduce_unit_slow(const FoCommArgs& A, int64_t off, int cnt, float2 (&g)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) g[i] = make_float2(0.f, 0.f);
  for (int p = 0; p < A.world; ++p) {
    Raw8<T> r;
    load_raw8_partial<T>(r, reinterpret_cast<const T*>(static_cast<const char*>(A.grad[p]) + off), cnt);
    float2 x[4];
    unpack8<T>(r, x);
#pragma unroll
    for (int i = 0; i < 4; ++i) g[i] = add2(g[i], x[i]);
  }
}


}  // namespace fo
