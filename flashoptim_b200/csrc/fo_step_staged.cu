// Bulk-copy staged variants of the fused steps (bf16 / fp16 parameters, 8-bit states).
// Same arithmetic as the reference's step kernels (flashoptim/optimizers.py:1587-1719,
// :2256-2443); the data path below has no counterpart there.
//
// The register-path kernels hold at most 32 warps x 56 B of loads in flight per
// SM and sit at about one eligible warp per scheduler.  Here a producer warp
// streams whole chunks (parameter, gradient, correction codes, state codes and
// their scales: 14-17 KB) into a ring of shared-memory stages with
// cp.async.bulk (the TMA unit's untiled copy; no multicast, no tensor map),
// completion is tracked by one mbarrier per stage, and eight consumer warps read
// their units from shared memory, release the stage and run the same update
// and stores as the register path.  Up to kStages - 1 chunks per CTA are in
// flight regardless of what the consumers are doing.
//
// A chunk that is not a full, 16-byte aligned 2048-element block (tails,
// tensors at odd offsets) skips the copy engine: the producer completes the
// stage's phase with a plain arrive and the consumers load it directly.
//
// Every mbarrier wait is bounded (wall clock); a wait that runs out records a
// code in StepParams.status (when given), and the waiting warp leaves its loop.
#include "fo_stage.cuh"
#include "fo_step_table.cuh"

namespace fo {

// Ring depth and CTAs per SM.  On the 291-tensor Llama-3-8B list 4 stages x 3 CTAs
// (9 chunks = 131 KB in flight per SM) measured best or within noise of the best for
// every kernel; deeper rings with 2 CTAs win on a single huge tensor but not on the
// list.  -DFO_STAGES / -DFO_STAGED_CTAS_PER_SM override both for tuning builds.
template <int kErr>
struct StageConfig {
#if defined(FO_STAGES) && defined(FO_STAGED_CTAS_PER_SM)
  static constexpr int kStages = FO_STAGES, kCtasPerSm = FO_STAGED_CTAS_PER_SM;
#else
  static constexpr int kStages = 4;
  static constexpr int kCtasPerSm = 3;
#endif
};
constexpr int kConsumerThreads = 256;
constexpr int kConsumerWarps = kConsumerThreads / 32;
constexpr int kStagedThreads = kConsumerThreads + 32;
constexpr int kStagedChunk = kConsumerThreads * kUnit;  // must equal kChunk of the table
static_assert(kStagedChunk == kChunk, "staged kernels share the chunk prefix of the register path");

template <int kErr, int kStates>
struct StageLayout {
  static constexpr int kP = 0;
  static constexpr int kG = kP + kStagedChunk * 2;
  static constexpr int kEcc = kG + kStagedChunk * 2;
  static constexpr int kQ0 = kEcc + kStagedChunk * kErr;
  static constexpr int kQ1 = kQ0 + kStagedChunk;
  static constexpr int kS0 = kQ0 + kStagedChunk * kStates;
  static constexpr int kS1 = kS0 + (kStagedChunk / kGroup) * 2;
  static constexpr int kBytes = kS0 + kStates * (kStagedChunk / kGroup) * 2;
  static constexpr int kStride = (kBytes + 127) / 128 * 128;
};

// A chunk goes through the copy engine when it is a full block of a segment whose
// streams (including the scale vectors) are 16-byte aligned.
__device__ __forceinline__ bool chunk_is_staged(const ChunkWalker& w, int c) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(w.S.s0s) | reinterpret_cast<uintptr_t>(w.S.s1s);
  const int64_t base = (int64_t)(c - w.seg_begin) * kStagedChunk;
  return w.vec && (a & 15) == 0 && base + kStagedChunk <= w.S.n;
}

template <typename T, int kErr, int kStates, typename Hyper, typename Update>
__device__ __forceinline__ void staged_body(const StepParams& P, const Hyper& H, Update update) {
  using L = StageLayout<kErr, kStates>;
  using Regs = UnitRegs<T, kErr, kStates, true>;
  constexpr int kStages = StageConfig<kErr>::kStages;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kStages], empty[kStages];

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    if (lane != 0) return;
    ChunkWalker w(P);
    int j = 0;
    for (int c = blockIdx.x; c < w.total; c += gridDim.x, ++j) {
      const int s = j % kStages;
      if (j >= kStages && !mbar_wait(&empty[s], ((j / kStages) - 1) & 1)) {
        if (P.status) atomicOr(P.status, 1u);
        return;
      }
      w.seek(c);
      if (!chunk_is_staged(w, c)) {
        mbar_arrive(&full[s]);
        continue;
      }
      const int64_t base = (int64_t)(c - w.seg_begin) * kStagedChunk;
      unsigned char* st = smem + s * L::kStride;
      mbar_arrive_expect_tx(&full[s], L::kBytes);
      bulk_load(st + L::kP, static_cast<const char*>(w.S.p) + base * 2, kStagedChunk * 2, &full[s]);
      bulk_load(st + L::kG, static_cast<const char*>(w.S.g) + base * 2, kStagedChunk * 2, &full[s]);
      if constexpr (kErr > 0)
        bulk_load(st + L::kEcc, static_cast<const char*>(w.S.ecc) + base * kErr, kStagedChunk * kErr, &full[s]);
      bulk_load(st + L::kQ0, static_cast<const char*>(w.S.s0) + base, kStagedChunk, &full[s]);
      bulk_load(st + L::kS0, static_cast<const char*>(w.S.s0s) + (base >> 5) * 2, (kStagedChunk / kGroup) * 2,
                &full[s]);
      if constexpr (kStates == 2) {
        bulk_load(st + L::kQ1, static_cast<const char*>(w.S.s1) + base, kStagedChunk, &full[s]);
        bulk_load(st + L::kS1, static_cast<const char*>(w.S.s1s) + (base >> 5) * 2, (kStagedChunk / kGroup) * 2,
                  &full[s]);
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  ChunkWalker w(P);
  int j = 0;
  for (int c = blockIdx.x; c < w.total; c += gridDim.x, ++j) {
    const int s = j % kStages;
    w.seek(c);
    const bool staged = chunk_is_staged(w, c);
    const int64_t base = (int64_t)(c - w.seg_begin) * kStagedChunk + (int64_t)threadIdx.x * kUnit;
    // one verdict per warp: at the deadline lanes may disagree, and the group shuffles in
    // store_unit need all 32 lanes
    if (!__all_sync(kFullMask, mbar_wait(&full[s], (j / kStages) & 1))) {
      if (P.status && lane == 0) atomicOr(P.status, 2u);
      return;
    }
    Regs r;
    if (staged) {
      const unsigned char* st = smem + s * L::kStride;
      r.cnt = kUnit;
      r.p.v = *reinterpret_cast<const uint4*>(st + L::kP + threadIdx.x * 16);
      r.g.v = *reinterpret_cast<const uint4*>(st + L::kG + threadIdx.x * 16);
      r.ecc = make_uint4(0, 0, 0, 0);
      if constexpr (kErr == 1) {
        const uint2 e = *reinterpret_cast<const uint2*>(st + L::kEcc + threadIdx.x * 8);
        r.ecc.x = e.x;
        r.ecc.y = e.y;
      } else if constexpr (kErr == 2) {
        r.ecc = *reinterpret_cast<const uint4*>(st + L::kEcc + threadIdx.x * 16);
      }
      r.q[0] = *reinterpret_cast<const uint2*>(st + L::kQ0 + threadIdx.x * 8);
      r.sc[0] = __half2float(*reinterpret_cast<const __half*>(st + L::kS0 + (threadIdx.x >> 2) * 2));
      if constexpr (kStates == 2) {
        r.q[1] = *reinterpret_cast<const uint2*>(st + L::kQ1 + threadIdx.x * 8);
        r.sc[1] = __half2float(*reinterpret_cast<const __half*>(st + L::kS1 + (threadIdx.x >> 2) * 2));
      }
    } else {
      load_unit_state(r, w.S, base, w.vec);
      load_unit_grad(r, w.S, base, w.vec);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);  // this warp holds its units in registers now
    float2 p[4], g[4], m[4], v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) m[i] = v[i] = make_float2(0.f, 0.f);
    unpack8<T>(r.g, g);
    widen_unit(r, p, m, v);
    update(p, g, m, v, H);
    store_unit(r, w.S, base, w.vec, p, m, v);
  }
}

struct AdamUpdate {
  __device__ __forceinline__ void operator()(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4], float2 (&v)[4],
                                             const FoAdamHyper& H) const {
    adam_update8<true>(p, g, m, v, H);
  }
};
struct MomentumUpdate {
  __device__ __forceinline__ void operator()(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4], float2 (&v)[4],
                                             const FoMomentumHyper& H) const {
    momentum_update8(p, g, m, H, true);
  }
};

template <typename T, int kErr>
__global__ void __launch_bounds__(kStagedThreads, StageConfig<kErr>::kCtasPerSm)
    adam_staged_kernel(const __grid_constant__ StepParams P, const __grid_constant__ FoAdamHyper H) {
  staged_body<T, kErr, 2>(P, H, AdamUpdate());
}
template <typename T, int kErr>
__global__ void __launch_bounds__(kStagedThreads, StageConfig<kErr>::kCtasPerSm)
    momentum_staged_kernel(const __grid_constant__ StepParams P, const __grid_constant__ FoMomentumHyper H) {
  staged_body<T, kErr, 1>(P, H, MomentumUpdate());
}

// Grid = resident CTAs x up to this factor: the hardware hands out the later CTAs as earlier
// ones finish, which evens out SMs that run at different paces (equal fixed shares wait for
// the slowest).  On the 291-tensor Llama-3-8B list, sustained under the power cap: AdamW-24
// 2.30 -> 2.24 ms per 1 B parameters, AdamW-32 2.54 -> 2.40, Lion-24 1.83 -> 1.78 for a factor of
// 6-12; 32 loses part of it again.  A CTA keeps at least kMinChunksPerCta chunks so that its
// ring fills: launches below about 60 M elements keep one round.
#ifndef FO_STAGED_ROUNDS
#define FO_STAGED_ROUNDS 8
#endif
static int g_staged_rounds = FO_STAGED_ROUNDS;
constexpr int kMinChunksPerCta = 16;

template <int kErr, int kStates, typename Kernel, typename Hyper>
static int launch_staged(Kernel kernel, const StepParams& P, const Hyper& H, int sm_count, cudaStream_t st) {
  constexpr int smem_bytes = StageConfig<kErr>::kStages * StageLayout<kErr, kStates>::kStride;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return (int)e;
  const int64_t resident = (int64_t)sm_count * StageConfig<kErr>::kCtasPerSm;
  int64_t rounds = P.total_chunks / (resident * kMinChunksPerCta);
  if (rounds > g_staged_rounds) rounds = g_staged_rounds;
  if (rounds < 1) rounds = 1;
  int64_t grid = resident * rounds;
  if (P.total_chunks < grid) grid = P.total_chunks;
  kernel<<<(int)grid, kStagedThreads, smem_bytes, st>>>(P, H);
  return (int)cudaGetLastError();
}

template <typename T>
static int staged_adam_t(const StepParams& P, const FoAdamHyper& H, int err, int sms, cudaStream_t st) {
  switch (err) {
    case 0: return launch_staged<0, 2>(adam_staged_kernel<T, 0>, P, H, sms, st);
    case 1: return launch_staged<1, 2>(adam_staged_kernel<T, 1>, P, H, sms, st);
    case 2: return launch_staged<2, 2>(adam_staged_kernel<T, 2>, P, H, sms, st);
  }
  return -1;
}
template <typename T>
static int staged_momentum_t(const StepParams& P, const FoMomentumHyper& H, int err, int sms, cudaStream_t st) {
  switch (err) {
    case 0: return launch_staged<0, 1>(momentum_staged_kernel<T, 0>, P, H, sms, st);
    case 1: return launch_staged<1, 1>(momentum_staged_kernel<T, 1>, P, H, sms, st);
    case 2: return launch_staged<2, 1>(momentum_staged_kernel<T, 2>, P, H, sms, st);
  }
  return -1;
}

int staged_adam_launch(const StepParams& P, const FoAdamHyper& H, int dtype, int err_bytes, int quantized,
                       int sm_count, cudaStream_t st) {
  if (!quantized) return -1;
  if (dtype == FO_BF16) return staged_adam_t<__nv_bfloat16>(P, H, err_bytes, sm_count, st);
  if (dtype == FO_FP16) return staged_adam_t<__half>(P, H, err_bytes, sm_count, st);
  return -1;
}

int staged_momentum_launch(const StepParams& P, const FoMomentumHyper& H, int dtype, int err_bytes,
                           int state_mode, int sm_count, cudaStream_t st) {
  if (state_mode != FO_STATE_Q8) return -1;
  if (dtype == FO_BF16) return staged_momentum_t<__nv_bfloat16>(P, H, err_bytes, sm_count, st);
  if (dtype == FO_FP16) return staged_momentum_t<__half>(P, H, err_bytes, sm_count, st);
  return -1;
}

}  // namespace fo

extern "C" void fo_set_staged_rounds(int rounds) { fo::g_staged_rounds = rounds < 1 ? 1 : (rounds > 1024 ? 1024 : rounds); }
extern "C" int fo_get_staged_rounds(void) { return fo::g_staged_rounds; }

