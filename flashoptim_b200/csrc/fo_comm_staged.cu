// Bulk-copy staged variant of the steps fused with the gradient collective (bf16 / fp16
// parameters, 8-bit states, peer loads).  No counterpart in the reference (NCCL reduce-scatter,
// then flashoptim/optimizers.py:2256-2443 per tensor).
//
// The register-path kernels of fo_comm.cu keep at most 8 x 16 bytes of remote requests in
// flight per thread, so saturating NVLink (770 GB/s x a few microseconds of latency = a few
// MB in flight) takes most of the GPU's threads, which backward's GEMMs then do not get.
// Here ONE producer thread per CTA asks the TMA unit for whole 2048-element chunks with
// cp.async.bulk (untiled, no tensor map, NO multicast of any kind): the W ranks' copies of
// the gradient chunk straight out of the peers' memory, and this rank's parameter,
// correction codes, state codes and scales, into a ring of shared-memory stages whose
// mbarriers count the bytes.  Eight consumer warps add the W copies in fp32 in rank order,
// run the same per-unit update as every other step kernel and store.  A CTA keeps
// (stages - 1) x W x 4 KB of remote data in flight without holding a register for it, so two
// or three dozen CTAs fill the links and the other SMs stay with the GEMMs.
//
// Chunks that are not full aligned blocks take the element-wise path inside the same kernel.
// Every wait (flags, mbarriers) is bounded; a wait that runs out records a bit in the status
// word, the CTA stops issuing copies, waits (bounded again) for the copies it still has in
// flight, and leaves without publishing "done".
#include "fo_comm.cuh"
#include "fo_stage.cuh"

namespace fo {

constexpr int kPsConsumerThreads = 256;
constexpr int kPsConsumerWarps = kPsConsumerThreads / 32;
constexpr int kPsThreads = kPsConsumerThreads + 32;
constexpr int kPsChunk = kPsConsumerThreads * kUnit;  // 2048 elements
constexpr int kPsScaleBytes = (kPsChunk / kGroup) * 2;
constexpr unsigned kPsProducerTimeout = 0x40000000u, kPsConsumerTimeout = 0x80000000u;

// Shared-memory image of one chunk: local streams first, then kW gradient copies.
template <int kErr, int kStates, int kW>
struct PeerStageLayout {
  static constexpr int kP = 0;
  static constexpr int kEcc = kP + kPsChunk * 2;
  static constexpr int kQ0 = kEcc + kPsChunk * kErr;
  static constexpr int kQ1 = kQ0 + kPsChunk;
  static constexpr int kS0 = kQ0 + kPsChunk * kStates;
  static constexpr int kS1 = kS0 + kPsScaleBytes;
  static constexpr int kLocalBytes = kS0 + kStates * kPsScaleBytes;
  static constexpr int kG = (kLocalBytes + 127) / 128 * 128;
  static constexpr int kStride = kG + kW * kPsChunk * 2;
  // ring depth: as many stages as fit into about 180 KB, at most 8
  static constexpr int kStages = (184320 / kStride) > 8 ? 8 : (184320 / kStride);
};

__device__ __forceinline__ bool ps_chunk_is_staged(const CommWalker& w, int c) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(w.S.s0s) | reinterpret_cast<uintptr_t>(w.S.s1s);
  const int64_t base = (int64_t)(c - w.seg_begin) * kPsChunk;
  return w.vec && (a & 15) == 0 && base + kPsChunk <= w.S.n;
}

// Bounded mbarrier wait with the collective's own limit.
__device__ __forceinline__ bool ps_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = now_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (now_ns() - t0 > limit_ns) return false;
  }
}

template <typename T, int kErr, int kStates, int kW, typename Hyper, typename Update>
__device__ __forceinline__ void peer_staged_body(const FoSeg* segs, const int32_t* cb, int total_chunks,
                                                 const Hyper& H, const FoCommArgs& A, Update update) {
  using L = PeerStageLayout<kErr, kStates, kW>;
  using Regs = UnitRegs<T, kErr, kStates, true>;
  constexpr int kStages = L::kStages;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kStages], empty[kStages];
  __shared__ int issued;     // chunks (of this CTA) whose copies the producer has requested
  __shared__ int abort_flag;  // a wait ran out somewhere in this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kPsConsumerWarps);
    }
    issued = 0;
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool started = start_barrier(A);  // whole CTA, includes a __syncthreads
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t limit = A.timeout_ns;

  if (started && warp == kPsConsumerWarps) {
    // ---------------------------------------------------------------- producer
    // Lane 0 waits and issues; the whole warp walks the loop so that it reaches the CTA
    // barrier below converged.
    CommWalker w(segs, cb);
    int j = 0;
    for (int c = blockIdx.x; c < total_chunks; c += gridDim.x, ++j) {
      const int s = j % kStages;
      int stop = 0;
      if (lane == 0) {
        if (*(volatile int*)&abort_flag) {
          stop = 1;
        } else if (j >= kStages && !ps_wait(&empty[s], ((j / kStages) - 1) & 1, limit)) {
          atomicOr(reinterpret_cast<unsigned int*>(A.status), kPsProducerTimeout);
          *(volatile int*)&abort_flag = 1;
          stop = 1;
        }
      }
      stop = __shfl_sync(kFullMask, stop, 0);
      if (stop) break;
      w.seek(c);
      if (lane == 0) {
        if (!ps_chunk_is_staged(w, c)) {
          mbar_arrive(&full[s]);
        } else {
          const int64_t base = (int64_t)(c - w.seg_begin) * kPsChunk;
          const int64_t goff = (int64_t)reinterpret_cast<intptr_t>(w.S.g) + base * 2;
          unsigned char* st = smem + s * L::kStride;
          mbar_arrive_expect_tx(&full[s], (uint32_t)(L::kLocalBytes + A.world * kPsChunk * 2));
          // the remote copies first: they have the longest way to go
          for (int p = 0; p < A.world; ++p)
            bulk_load(st + L::kG + p * (kPsChunk * 2), static_cast<const char*>(A.grad[p]) + goff, kPsChunk * 2,
                      &full[s]);
          bulk_load(st + L::kP, static_cast<const char*>(w.S.p) + base * 2, kPsChunk * 2, &full[s]);
          if constexpr (kErr > 0)
            bulk_load(st + L::kEcc, static_cast<const char*>(w.S.ecc) + base * kErr, kPsChunk * kErr, &full[s]);
          if constexpr (kStates >= 1) {
            bulk_load(st + L::kQ0, static_cast<const char*>(w.S.s0) + base, kPsChunk, &full[s]);
            bulk_load(st + L::kS0, static_cast<const char*>(w.S.s0s) + (base >> 5) * 2, kPsScaleBytes, &full[s]);
          }
          if constexpr (kStates == 2) {
            bulk_load(st + L::kQ1, static_cast<const char*>(w.S.s1) + base, kPsChunk, &full[s]);
            bulk_load(st + L::kS1, static_cast<const char*>(w.S.s1s) + (base >> 5) * 2, kPsScaleBytes, &full[s]);
          }
        }
        *(volatile int*)&issued = j + 1;
      }
      __syncwarp();
    }
  } else if (started) {
    // ------------------------------------------------------------------ consumers
    CommWalker w(segs, cb);
    int j = 0;
    for (int c = blockIdx.x; c < total_chunks; c += gridDim.x, ++j) {
      const int s = j % kStages;
      w.seek(c);
      const bool staged = ps_chunk_is_staged(w, c);
      const int64_t base = (int64_t)(c - w.seg_begin) * kPsChunk + (int64_t)threadIdx.x * kUnit;
      const int64_t off = (int64_t)reinterpret_cast<intptr_t>(w.S.g) + base * (int64_t)sizeof(T);
      // one verdict per warp: the group shuffles of store_unit need all 32 lanes
      if (!__all_sync(kFullMask, ps_wait(&full[s], (j / kStages) & 1, limit))) {
        if (lane == 0) {
          atomicOr(reinterpret_cast<unsigned int*>(A.status), kPsConsumerTimeout);
          *(volatile int*)&abort_flag = 1;
        }
        break;
      }
      Regs r;
      float2 g[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) g[i] = make_float2(0.f, 0.f);
      if (staged) {
        const unsigned char* st = smem + s * L::kStride;
        r.cnt = kUnit;
        r.p.v = *reinterpret_cast<const uint4*>(st + L::kP + threadIdx.x * 16);
        r.ecc = make_uint4(0, 0, 0, 0);
        if constexpr (kErr == 1) {
          const uint2 e = *reinterpret_cast<const uint2*>(st + L::kEcc + threadIdx.x * 8);
          r.ecc.x = e.x;
          r.ecc.y = e.y;
        } else if constexpr (kErr == 2) {
          r.ecc = *reinterpret_cast<const uint4*>(st + L::kEcc + threadIdx.x * 16);
        }
        if constexpr (kStates >= 1) {
          r.q[0] = *reinterpret_cast<const uint2*>(st + L::kQ0 + threadIdx.x * 8);
          r.sc[0] = __half2float(*reinterpret_cast<const __half*>(st + L::kS0 + (threadIdx.x >> 2) * 2));
        }
        if constexpr (kStates == 2) {
          r.q[1] = *reinterpret_cast<const uint2*>(st + L::kQ1 + threadIdx.x * 8);
          r.sc[1] = __half2float(*reinterpret_cast<const __half*>(st + L::kS1 + (threadIdx.x >> 2) * 2));
        }
#pragma unroll
        for (int p = 0; p < kW; ++p) {
          if (p < A.world) {  // fp32 sum in rank order: every replica adds in the same order
            Raw8<T> x;
            x.v = *reinterpret_cast<const uint4*>(st + L::kG + p * (kPsChunk * 2) + threadIdx.x * 16);
            float2 xf[4];
            unpack8<T>(x, xf);
#pragma unroll
            for (int i = 0; i < 4; ++i) g[i] = add2(g[i], xf[i]);
          }
        }
      } else {
        load_unit_state(r, w.S, base, w.vec);
        if (r.cnt == kUnit && w.vec) {
          Raw8<T> x[kW];
#pragma unroll
          for (int p = 0; p < kW; ++p)
            if (p < A.world)
              load_raw8<T>(x[p], reinterpret_cast<const T*>(static_cast<const char*>(A.grad[p]) + off), true);
#pragma unroll
          for (int p = 0; p < kW; ++p) {
            if (p < A.world) {
              float2 xf[4];
              unpack8<T>(x[p], xf);
#pragma unroll
              for (int i = 0; i < 4; ++i) g[i] = add2(g[i], xf[i]);
            }
          }
        } else if (r.cnt > 0) {
          reduce_unit_slow<T>(A, off, r.cnt, g);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);  // this warp holds its units in registers now
      const bool vec = w.vec && r.cnt == kUnit;
      float2 p[4], m[4], v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) m[i] = v[i] = make_float2(0.f, 0.f);
      store_grad_out<T>(A, off, r.cnt, vec, g, H.grad_scale);
      widen_unit(r, p, m, v);
      update(p, g, m, v, H);
      Raw8<T> pn;
      store_unit(r, w.S, base, w.vec, p, m, v, pn);
      if (A.push) push_param<T, FO_MAX_PEERS>(A, off, r.cnt, vec, pn);
    }
  }
  __syncthreads();
  const bool completed = started && abort_flag == 0;
  if (!completed && threadIdx.x == 0) {
    // copies that were requested but never consumed must land before this CTA's shared
    // memory goes to somebody else: wait for each stage's newest phase, within the limit
    const int n = issued;
    for (int s = 0; s < kStages && s < n; ++s) {
      const int j = ((n - 1 - s) / kStages) * kStages + s;  // newest issued chunk on stage s
      ps_wait(&full[s], (j / kStages) & 1, limit);
    }
  }
  end_signal(A, 2, false, completed);
}

template <bool kHasState>
struct PsMomentumUpdate {
  __device__ __forceinline__ void operator()(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4], float2 (&v)[4],
                                             const FoMomentumHyper& H) const {
    momentum_update8(p, g, m, H, kHasState);
  }
};
struct PsAdamUpdate {
  __device__ __forceinline__ void operator()(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4], float2 (&v)[4],
                                             const FoAdamHyper& H) const {
    adam_update8<true>(p, g, m, v, H);
  }
};

template <typename T, int kErr, int kW>
__global__ void __launch_bounds__(kPsThreads, 1)
    adam_peer_staged_kernel(const FoSeg* __restrict__ segs, const int32_t* __restrict__ cb, int total_chunks,
                            const __grid_constant__ FoAdamHyper H, const __grid_constant__ FoCommArgs A) {
  peer_staged_body<T, kErr, 2, kW>(segs, cb, total_chunks, H, A, PsAdamUpdate());
}
template <typename T, int kErr, int kW>
__global__ void __launch_bounds__(kPsThreads, 1)
    momentum_peer_staged_kernel(const FoSeg* __restrict__ segs, const int32_t* __restrict__ cb, int total_chunks,
                                const __grid_constant__ FoMomentumHyper H, const __grid_constant__ FoCommArgs A) {
  peer_staged_body<T, kErr, 1, kW>(segs, cb, total_chunks, H, A, PsMomentumUpdate<true>());
}

template <int kErr, int kStates, int kW, typename Kernel, typename Hyper>
static int launch_ps(Kernel kernel, const FoSeg* s, const int32_t* cb, int total, const Hyper& H,
                     const FoCommArgs& A, int grid, cudaStream_t st) {
  using L = PeerStageLayout<kErr, kStates, kW>;
  constexpr int smem_bytes = L::kStages * L::kStride;
  static_assert(L::kStages >= 2, "the ring needs at least two stages");
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  kernel<<<grid, kPsThreads, smem_bytes, st>>>(s, cb, total, H, A);
  return (int)cudaGetLastError();
}

template <typename T, int kErr>
static int ps_adam_w(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H, const FoCommArgs& A,
                     int grid, cudaStream_t st) {
  if (A.world <= 2) return launch_ps<kErr, 2, 2>(adam_peer_staged_kernel<T, kErr, 2>, s, cb, total, H, A, grid, st);
  if (A.world <= 4) return launch_ps<kErr, 2, 4>(adam_peer_staged_kernel<T, kErr, 4>, s, cb, total, H, A, grid, st);
  return launch_ps<kErr, 2, 8>(adam_peer_staged_kernel<T, kErr, 8>, s, cb, total, H, A, grid, st);
}
template <typename T, int kErr>
static int ps_mom_w(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H, const FoCommArgs& A,
                    int grid, cudaStream_t st) {
  if (A.world <= 2)
    return launch_ps<kErr, 1, 2>(momentum_peer_staged_kernel<T, kErr, 2>, s, cb, total, H, A, grid, st);
  if (A.world <= 4)
    return launch_ps<kErr, 1, 4>(momentum_peer_staged_kernel<T, kErr, 4>, s, cb, total, H, A, grid, st);
  return launch_ps<kErr, 1, 8>(momentum_peer_staged_kernel<T, kErr, 8>, s, cb, total, H, A, grid, st);
}

template <typename T>
static int ps_adam_t(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H, const FoCommArgs& A,
                     int err, int grid, cudaStream_t st) {
  switch (err) {
    case 0: return ps_adam_w<T, 0>(s, cb, total, H, A, grid, st);
    case 1: return ps_adam_w<T, 1>(s, cb, total, H, A, grid, st);
    case 2: return ps_adam_w<T, 2>(s, cb, total, H, A, grid, st);
  }
  return -1;
}
template <typename T>
static int ps_mom_t(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H, const FoCommArgs& A,
                    int err, int grid, cudaStream_t st) {
  switch (err) {
    case 0: return ps_mom_w<T, 0>(s, cb, total, H, A, grid, st);
    case 1: return ps_mom_w<T, 1>(s, cb, total, H, A, grid, st);
    case 2: return ps_mom_w<T, 2>(s, cb, total, H, A, grid, st);
  }
  return -1;
}

// One CTA per SM at most (the ring takes most of an SM's shared memory).
static int ps_grid(int total, const FoCommArgs& A) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  int g = sms;
  if (A.max_ctas > 0 && A.max_ctas < g) g = A.max_ctas;
  if (total < g) g = total;
  return g < 1 ? 1 : g;
}

// Return -1 when the combination is not served by a staged kernel.
int staged_adam_peer_launch(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                            const FoCommArgs& A, int dtype, int err_bytes, int quantized, cudaStream_t st) {
  if (!quantized || A.multicast != nullptr) return -1;
  const int grid = ps_grid(total, A);
  if (dtype == FO_BF16) return ps_adam_t<__nv_bfloat16>(s, cb, total, H, A, err_bytes, grid, st);
  if (dtype == FO_FP16) return ps_adam_t<__half>(s, cb, total, H, A, err_bytes, grid, st);
  return -1;
}
int staged_momentum_peer_launch(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                                const FoCommArgs& A, int dtype, int err_bytes, int state_mode, cudaStream_t st) {
  if (state_mode != FO_STATE_Q8 || A.multicast != nullptr) return -1;
  const int grid = ps_grid(total, A);
  if (dtype == FO_BF16) return ps_mom_t<__nv_bfloat16>(s, cb, total, H, A, err_bytes, grid, st);
  if (dtype == FO_FP16) return ps_mom_t<__half>(s, cb, total, H, A, err_bytes, grid, st);
  return -1;
}

}  // namespace fo
