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
#include "fo_comm.cuh"

namespace fo {

// Units per thread and remote copies per unit.  With peer loads a unit issues one 16-byte
// request per rank, so the fewer ranks, the more units a thread puts in flight (2 ranks: 4
// units, 3-4 ranks: 2, 5-8 ranks: 1; eight requests per thread either way).  With
// multimem.ld_reduce a unit is ONE request whatever the world size (the switch adds the
// ranks' copies), so a thread always takes 4 units: the kernel is bound by NVLink latency
// times bytes in flight, and the more a CTA keeps in flight, the fewer CTAs (SMs taken
// from backward's GEMMs) saturate the links.
template <int kU, bool kMc>
struct PeerCfg {
  static constexpr int kPeers = kMc ? 1 : FO_MAX_PEERS / kU;  // register slots per unit
  static constexpr int kChunk = kCommThreads * kUnit * kU;
  static constexpr int kCtas = 2;  // 128 registers per thread: no variant of bf16 / fp16 spills
};

template <typename T, int kErr, int kStates, bool kQ, int kU, bool kMc, typename Hyper, typename Update>
__device__ __forceinline__ void peer_step_body(const FoSeg* segs, const int32_t* cb, int total_chunks,
                                               const Hyper& H, const FoCommArgs& A, Update update) {
  using Regs = UnitRegs<T, kErr, kStates, kQ>;
  using Cfg = PeerCfg<kU, kMc>;
  constexpr int kPeers = Cfg::kPeers;
  CommWalker w(segs, cb);
  for (int c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    w.seek(c);
    const int64_t chunk_base = (int64_t)(c - w.seg_begin) * Cfg::kChunk;
    const int64_t g0 = (int64_t)reinterpret_cast<intptr_t>(w.S.g);
    Raw8<T> remote[kU][kPeers];
    // phase 1: request the remote copies of every full, aligned unit of this thread
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t base = chunk_base + (int64_t)(u * kCommThreads + threadIdx.x) * kUnit;
      if (w.vec && w.S.n - base >= kUnit) {
        const int64_t off = g0 + base * (int64_t)sizeof(T);
        if constexpr (kMc) {
          const char* a = static_cast<const char*>(A.multicast) + off;
          if constexpr (sizeof(T) == 4) {
            remote[u][0].v = multimem_ld_reduce_f32x4(a);
            remote[u][0].w = multimem_ld_reduce_f32x4(a + 16);
          } else if constexpr (Elem<T>::kMant == 7) {
            remote[u][0].v = multimem_ld_reduce_bf16x8(a);
          } else {
            remote[u][0].v = multimem_ld_reduce_f16x8(a);
          }
        } else {
#pragma unroll
          for (int p = 0; p < kPeers; ++p)
            if (p < A.world)
              load_raw8<T>(remote[u][p], reinterpret_cast<const T*>(static_cast<const char*>(A.grad[p]) + off), true);
        }
      }
    }
    // phase 2: local state, sum, update, store (and push)
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t base = chunk_base + (int64_t)(u * kCommThreads + threadIdx.x) * kUnit;
      const int64_t off = g0 + base * (int64_t)sizeof(T);
      Regs r;
      load_unit_state(r, w.S, base, w.vec);
      const bool vec = w.vec && r.cnt == kUnit;
      float2 p[4], g[4], m[4], v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) g[i] = m[i] = v[i] = make_float2(0.f, 0.f);
      if (vec) {
        if constexpr (kMc) {
          unpack8<T>(remote[u][0], g);
        } else {
#pragma unroll
          for (int q = 0; q < kPeers; ++q) {
            if (q < A.world) {  // fp32 sum in rank order: every replica adds in the same order
              float2 x[4];
              unpack8<T>(remote[u][q], x);
#pragma unroll
              for (int i = 0; i < 4; ++i) g[i] = add2(g[i], x[i]);
            }
          }
        }
      } else if (r.cnt > 0) {
        reduce_unit_slow<T>(A, off, r.cnt, g);
      }
      store_grad_out<T>(A, off, r.cnt, vec, g, H.grad_scale);
      widen_unit(r, p, m, v);
      update(p, g, m, v, H);
      Raw8<T> pn;
      store_unit(r, w.S, base, w.vec, p, m, v, pn);
      if (A.push) push_param<T, FO_MAX_PEERS>(A, off, r.cnt, vec, pn);
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

template <typename T, int kErr, bool kQ, int kU, bool kMc>
__global__ void __launch_bounds__(kCommThreads, PeerCfg<kU, kMc>::kCtas)
    adam_peer_kernel(const FoSeg* __restrict__ segs, const int32_t* __restrict__ cb, int total_chunks,
                     const __grid_constant__ FoAdamHyper H, const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) {
    end_signal(A, 2, false, false);
    return;
  }
  peer_step_body<T, kErr, 2, kQ, kU, kMc>(segs, cb, total_chunks, H, A, PeerAdamUpdate<kQ>());
  end_signal(A);
}

template <typename T, int kErr, int kMode, int kU, bool kMc>
__global__ void __launch_bounds__(kCommThreads, PeerCfg<kU, kMc>::kCtas)
    momentum_peer_kernel(const FoSeg* __restrict__ segs, const int32_t* __restrict__ cb, int total_chunks,
                         const __grid_constant__ FoMomentumHyper H, const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) {
    end_signal(A, 2, false, false);
    return;
  }
  constexpr int kStates = kMode == FO_STATE_NONE ? 0 : 1;
  constexpr bool kQ = kMode == FO_STATE_Q8;
  peer_step_body<T, kErr, kStates, kQ, kU, kMc>(segs, cb, total_chunks, H, A, PeerMomentumUpdate<(kStates > 0)>());
  end_signal(A);
}

// One CTA: publish this rank's arrival on the ready channel and wait (bounded) for every
// rank's.  Launched in front of a step kernel on the same stream, so that the many CTAs of
// the step kernel find the flags already set instead of occupying SMs while a slower rank
// is still packing its gradients.
__global__ void ready_barrier_kernel(const __grid_constant__ FoCommArgs A) {
  if (threadIdx.x < A.world) {
    __threadfence_system();
    st_release_sys(A.pad[threadIdx.x] + A.ready_channel * FO_MAX_PEERS + A.rank, A.epoch);
    wait_flag(A, A.ready_channel, threadIdx.x, A.epoch);
  }
}

// Plain averaged reduce (no update): out[i] = scale * sum_r peer_r[off + i].
// DDP buckets that must hand reduced gradients back, and the baseline for the
// fused kernels' comparisons.
template <typename T>
__global__ void __launch_bounds__(kCommThreads, kCommCtasPerSm)
    reduce_peer_kernel(int64_t n, int64_t src_off, T* __restrict__ out, float scale,
                       const __grid_constant__ FoCommArgs A) {
  if (!start_barrier(A)) {
    end_signal(A, 2, false, false);
    return;
  }
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
  if (!start_barrier(A)) {
    end_signal(A, 2, true, false);
    return;
  }
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
  if (!start_barrier(A)) {
    end_signal(A, 3, false, false);
    return;
  }
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

static int units_for_world(int world, bool multicast) {
  if (multicast) return 4;
  return world <= 2 ? 4 : (world <= 4 ? 2 : 1);
}

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

// The one-CTA barrier in front of a step kernel (see ready_barrier_kernel).
static void launch_ready_barrier(const FoCommArgs& A, cudaStream_t st) {
  if (A.world > 1 && !(A.flags & FO_COMM_NO_BARRIER)) ready_barrier_kernel<<<1, 32, 0, st>>>(A);
}

template <typename T, int kErr, int kU, bool kMc>
static int launch_adam_peer_q(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                              const FoCommArgs& A, int quantized, cudaStream_t st) {
  const int grid = comm_grid(total, &A, PeerCfg<kU, kMc>::kCtas);
  launch_ready_barrier(A, st);
  if (quantized) adam_peer_kernel<T, kErr, true, kU, kMc><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
  else adam_peer_kernel<T, kErr, false, kU, kMc><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
  return (int)cudaGetLastError();
}
template <typename T, int kErr>
static int launch_adam_peer_u(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                              const FoCommArgs& A, int quantized, cudaStream_t st) {
  if (A.multicast != nullptr) return launch_adam_peer_q<T, kErr, 4, true>(s, cb, total, H, A, quantized, st);
  switch (units_for_world(A.world, false)) {
    case 4: return launch_adam_peer_q<T, kErr, 4, false>(s, cb, total, H, A, quantized, st);
    case 2: return launch_adam_peer_q<T, kErr, 2, false>(s, cb, total, H, A, quantized, st);
  }
  return launch_adam_peer_q<T, kErr, 1, false>(s, cb, total, H, A, quantized, st);
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

template <typename T, int kErr, int kU, bool kMc>
static int launch_mom_peer_m(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                             const FoCommArgs& A, int mode, cudaStream_t st) {
  const int grid = comm_grid(total, &A, PeerCfg<kU, kMc>::kCtas);
  if (mode != FO_STATE_NONE && mode != FO_STATE_Q8 && mode != FO_STATE_FULL) return (int)cudaErrorInvalidValue;
  launch_ready_barrier(A, st);
  switch (mode) {
    case FO_STATE_NONE:
      momentum_peer_kernel<T, kErr, FO_STATE_NONE, kU, kMc><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
      break;
    case FO_STATE_Q8:
      momentum_peer_kernel<T, kErr, FO_STATE_Q8, kU, kMc><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
      break;
    default:
      momentum_peer_kernel<T, kErr, FO_STATE_FULL, kU, kMc><<<grid, kCommThreads, 0, st>>>(s, cb, total, H, A);
      break;
  }
  return (int)cudaGetLastError();
}
template <typename T, int kErr>
static int launch_mom_peer_u(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                             const FoCommArgs& A, int mode, cudaStream_t st) {
  if (A.multicast != nullptr) return launch_mom_peer_m<T, kErr, 4, true>(s, cb, total, H, A, mode, st);
  switch (units_for_world(A.world, false)) {
    case 4: return launch_mom_peer_m<T, kErr, 4, false>(s, cb, total, H, A, mode, st);
    case 2: return launch_mom_peer_m<T, kErr, 2, false>(s, cb, total, H, A, mode, st);
  }
  return launch_mom_peer_m<T, kErr, 1, false>(s, cb, total, H, A, mode, st);
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

namespace fo {
// fo_comm_staged.cu; -1 when the combination is not served by a staged kernel
int staged_adam_peer_launch(const FoSeg* s, const int32_t* cb, int total, const FoAdamHyper& H,
                            const FoCommArgs& A, int dtype, int err_bytes, int quantized, cudaStream_t st);
int staged_momentum_peer_launch(const FoSeg* s, const int32_t* cb, int total, const FoMomentumHyper& H,
                                const FoCommArgs& A, int dtype, int err_bytes, int state_mode, cudaStream_t st);

static bool use_staged(const FoCommArgs& A, int dtype, int q8_states) {
  return A.variant == 1 && A.multicast == nullptr && q8_states && (dtype == FO_BF16 || dtype == FO_FP16);
}
}  // namespace fo

extern "C" int fo_comm_step_chunk_elems(const FoCommArgs* comm, int dtype, int q8_states) {
  if (!comm) return fo::kCommChunk;
  if (fo::use_staged(*comm, dtype, q8_states)) return fo::kCommChunk;  // 2048: one unit per consumer thread
  return fo::kCommChunk * fo::units_for_world(comm->world, comm->multicast != nullptr);
}

extern "C" int fo_adam_step_peer(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                                 int dtype, int err_bytes, int quantized, const FoAdamHyper* hyper,
                                 const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm) || !hyper) return (int)cudaErrorInvalidValue;
  if (n_seg <= 0 || total_chunks <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (fo::use_staged(*comm, dtype, quantized)) {
    fo::launch_ready_barrier(*comm, st);
    return fo::staged_adam_peer_launch(segs, chunk_begin, total_chunks, *hyper, *comm, dtype, err_bytes, quantized,
                                       st);
  }
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
  if (fo::use_staged(*comm, dtype, state_mode == FO_STATE_Q8)) {
    fo::launch_ready_barrier(*comm, st);
    return fo::staged_momentum_peer_launch(segs, chunk_begin, total_chunks, *hyper, *comm, dtype, err_bytes,
                                           state_mode, st);
  }
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

extern "C" int fo_comm_barrier(const FoCommArgs* comm, void* stream) {
  if (!fo::args_ok(comm)) return (int)cudaErrorInvalidValue;
  fo::ready_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(*comm);
  return (int)cudaGetLastError();
}

extern "C" int fo_memcpy_async(void* dst, const void* src, int64_t nbytes, void* stream) {
  if (nbytes < 0 || (nbytes > 0 && (!dst || !src))) return (int)cudaErrorInvalidValue;
  if (nbytes == 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
}
