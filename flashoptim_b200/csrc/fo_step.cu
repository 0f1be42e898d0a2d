// Multi-tensor fused optimizer steps for sm_100a.
//
// One launch updates every tensor of a parameter group: a persistent grid of
// CTAs walks a list of "chunks" (kChunk consecutive elements of one tensor),
// so a Llama-sized parameter list costs one launch instead of one per tensor
// (the reference launches once per tensor: flashoptim/optimizers.py:1556-1579,
// :2226-2251) and 4096-element norm weights ride along with the big matrices.
// Each element makes one trip: gradient, parameter, correction codes and 8-bit
// moments are read once, the update runs in fp32 registers, and parameter,
// correction and requantised moments are written once
// (what flashoptim/optimizers.py:2255-2438 and :1586-1719 compute).
#include "fo_step_table.cuh"

namespace fo {

// Occupancy (4 CTAs of 256 threads at 64 registers), not register-level software
// prefetch, hides the memory latency here: a double-buffered variant of this loop
// measured slower on B200 at every occupancy that its extra registers allowed.
template <typename Regs, typename Load, typename Compute>
__device__ __forceinline__ void walk_chunks(ChunkWalker& w, Load load, Compute compute) {
  for (int c = blockIdx.x; c < w.total; c += gridDim.x) {
    w.seek(c);
    Regs r[kUnroll];
    load(r, c);
    compute(r, c);
  }
}

template <typename T, int kErr, bool kQ>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
    adam_kernel(const __grid_constant__ StepParams P, const __grid_constant__ FoAdamHyper H) {
  using Regs = UnitRegs<T, kErr, 2, kQ>;
  ChunkWalker w(P);
  walk_chunks<Regs>(
      w,
      [&](Regs(&r)[kUnroll], int c) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int64_t base = w.unit_base(c, u);
          load_unit_state(r[u], w.S, base, w.vec);
          load_unit_grad(r[u], w.S, base, w.vec);
        }
      },
      [&](Regs(&r)[kUnroll], int c) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int64_t base = w.unit_base(c, u);
          float2 p[4], g[4], m[4], v[4];
          unpack8<T>(r[u].g, g);
          widen_unit(r[u], p, m, v);
          adam_update8<kQ>(p, g, m, v, H);
          store_unit(r[u], w.S, base, w.vec, p, m, v);
        }
      });
}

template <typename T, int kErr, int kMode>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
    momentum_kernel(const __grid_constant__ StepParams P, const __grid_constant__ FoMomentumHyper H) {
  constexpr int kStates = kMode == FO_STATE_NONE ? 0 : 1;
  constexpr bool kQ = kMode == FO_STATE_Q8;
  using Regs = UnitRegs<T, kErr, kStates, kQ>;
  ChunkWalker w(P);
  walk_chunks<Regs>(
      w,
      [&](Regs(&r)[kUnroll], int c) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int64_t base = w.unit_base(c, u);
          load_unit_state(r[u], w.S, base, w.vec);
          load_unit_grad(r[u], w.S, base, w.vec);
        }
      },
      [&](Regs(&r)[kUnroll], int c) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int64_t base = w.unit_base(c, u);
          float2 p[4], g[4], m[4], v[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) m[i] = v[i] = make_float2(0.f, 0.f);
          unpack8<T>(r[u].g, g);
          widen_unit(r[u], p, m, v);
          momentum_update8(p, g, m, H, kStates > 0);
          store_unit(r[u], w.S, base, w.vec, p, m, v);
        }
      });
}

// ---------------------------------------------------------------- host side

static int g_sm_count[64];

static int sm_count(int device) {
  if (device < 0 || device >= 64) return 148;
  if (g_sm_count[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[device] = n;
  }
  return g_sm_count[device];
}

// 0: register-path kernels only; 1: bulk-copy staged kernels where they apply
static int g_step_variant = 1;
static unsigned int* g_status[64];

static int fill_params(StepParams& P, const FoSeg* segs, const int32_t* chunk_begin, int n_seg,
                       int total_chunks, int table_on_device) {
  P.n_seg = n_seg;
  P.total_chunks = total_chunks;
  int dev = 0;
  cudaGetDevice(&dev);
  P.status = (dev >= 0 && dev < 64) ? g_status[dev] : nullptr;
  if (table_on_device) {
    P.segs = segs;
    P.chunk_begin = chunk_begin;
    return 0;
  }
  if (n_seg > FO_MAX_INLINE_SEGS) return (int)cudaErrorInvalidValue;
  P.segs = nullptr;
  P.chunk_begin = nullptr;
  for (int i = 0; i < n_seg; ++i) P.inl.segs[i] = segs[i];
  for (int i = 0; i <= n_seg; ++i) P.inl.chunk_begin[i] = chunk_begin[i];
  for (int i = n_seg + 1; i <= FO_MAX_INLINE_SEGS; ++i) P.inl.chunk_begin[i] = total_chunks;
  return 0;
}

template <typename T, int kErr>
static int launch_adam_q(const StepParams& P, const FoAdamHyper& H, int quantized, int grid, cudaStream_t st) {
  if (quantized) adam_kernel<T, kErr, true><<<grid, kThreads, 0, st>>>(P, H);
  else adam_kernel<T, kErr, false><<<grid, kThreads, 0, st>>>(P, H);
  return (int)cudaGetLastError();
}
template <typename T>
static int launch_adam_e(const StepParams& P, const FoAdamHyper& H, int err, int quantized, int grid,
                         cudaStream_t st) {
  if constexpr (Elem<T>::kNarrow) {
    if (err == 1) return launch_adam_q<T, 1>(P, H, quantized, grid, st);
    if (err == 2) return launch_adam_q<T, 2>(P, H, quantized, grid, st);
  }
  if (err != 0) return (int)cudaErrorInvalidValue;
  return launch_adam_q<T, 0>(P, H, quantized, grid, st);
}

template <typename T, int kErr>
static int launch_mom_m(const StepParams& P, const FoMomentumHyper& H, int mode, int grid, cudaStream_t st) {
  switch (mode) {
    case FO_STATE_NONE: momentum_kernel<T, kErr, FO_STATE_NONE><<<grid, kThreads, 0, st>>>(P, H); break;
    case FO_STATE_Q8: momentum_kernel<T, kErr, FO_STATE_Q8><<<grid, kThreads, 0, st>>>(P, H); break;
    case FO_STATE_FULL: momentum_kernel<T, kErr, FO_STATE_FULL><<<grid, kThreads, 0, st>>>(P, H); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}
template <typename T>
static int launch_mom_e(const StepParams& P, const FoMomentumHyper& H, int err, int mode, int grid,
                        cudaStream_t st) {
  if constexpr (Elem<T>::kNarrow) {
    if (err == 1) return launch_mom_m<T, 1>(P, H, mode, grid, st);
    if (err == 2) return launch_mom_m<T, 2>(P, H, mode, grid, st);
  }
  if (err != 0) return (int)cudaErrorInvalidValue;
  return launch_mom_m<T, 0>(P, H, mode, grid, st);
}

static int grid_for(int total_chunks) {
  int dev = 0;
  cudaGetDevice(&dev);
  int g = sm_count(dev) * kCtasPerSm;
  return total_chunks < g ? total_chunks : g;
}

}  // namespace fo

extern "C" int fo_chunk_elems(void) { return fo::kChunk; }

extern "C" void fo_set_step_variant(int variant) { fo::g_step_variant = variant; }
extern "C" int fo_get_step_variant(void) { return fo::g_step_variant; }
extern "C" int fo_set_step_status(void* device_word) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  fo::g_status[dev] = static_cast<unsigned int*>(device_word);
  return 0;
}

extern "C" int fo_step_grid(int device) { return fo::sm_count(device) * fo::kCtasPerSm; }

extern "C" int fo_adam_step(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                            int table_on_device, int dtype, int err_bytes, int quantized,
                            const FoAdamHyper* hyper, void* stream) {
  if (n_seg <= 0 || total_chunks <= 0) return 0;
  fo::StepParams P;
  int rc = fo::fill_params(P, segs, chunk_begin, n_seg, total_chunks, table_on_device);
  if (rc) return rc;
  const int grid = fo::grid_for(total_chunks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (fo::g_step_variant == 1) {
    int dev = 0;
    cudaGetDevice(&dev);
    rc = fo::staged_adam_launch(P, *hyper, dtype, err_bytes, quantized, fo::sm_count(dev), st);
    if (rc != -1) return rc;
  }
  switch (dtype) {
    case FO_BF16: return fo::launch_adam_e<__nv_bfloat16>(P, *hyper, err_bytes, quantized, grid, st);
    case FO_FP16: return fo::launch_adam_e<__half>(P, *hyper, err_bytes, quantized, grid, st);
    case FO_FP32: return fo::launch_adam_e<float>(P, *hyper, err_bytes, quantized, grid, st);
  }
  return (int)cudaErrorInvalidValue;
}

extern "C" int fo_momentum_step(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                                int table_on_device, int dtype, int err_bytes, int state_mode,
                                const FoMomentumHyper* hyper, void* stream) {
  if (n_seg <= 0 || total_chunks <= 0) return 0;
  fo::StepParams P;
  int rc = fo::fill_params(P, segs, chunk_begin, n_seg, total_chunks, table_on_device);
  if (rc) return rc;
  const int grid = fo::grid_for(total_chunks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (fo::g_step_variant == 1) {
    int dev = 0;
    cudaGetDevice(&dev);
    rc = fo::staged_momentum_launch(P, *hyper, dtype, err_bytes, state_mode, fo::sm_count(dev), st);
    if (rc != -1) return rc;
  }
  switch (dtype) {
    case FO_BF16: return fo::launch_mom_e<__nv_bfloat16>(P, *hyper, err_bytes, state_mode, grid, st);
    case FO_FP16: return fo::launch_mom_e<__half>(P, *hyper, err_bytes, state_mode, grid, st);
    case FO_FP32: return fo::launch_mom_e<float>(P, *hyper, err_bytes, state_mode, grid, st);
  }
  return (int)cudaErrorInvalidValue;
}
