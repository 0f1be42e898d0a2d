// Launch configuration, segment table and chunk walker shared by the step kernels.
//
// No counterpart in the reference, which launches one Triton kernel per parameter tensor
// (flashoptim/optimizers.py:1535-1583, :2203-2252; grid from _make_grid, :2984-2996): here one
// launch walks a table of all tensors of a step.
#pragma once

#include "fo_step_core.cuh"

namespace fo {

#ifndef FO_UNROLL
#define FO_UNROLL 1
#endif
#ifndef FO_CTAS_PER_SM
#define FO_CTAS_PER_SM 4
#endif
#ifndef FO_THREADS
#define FO_THREADS 256
#endif
constexpr int kThreads = FO_THREADS;
constexpr int kUnroll = FO_UNROLL;  // units per thread per chunk; all loads of a chunk are issued before any math
constexpr int kChunk = kThreads * kUnit * kUnroll;
constexpr int kCtasPerSm = FO_CTAS_PER_SM;

struct InlineTable {
  FoSeg segs[FO_MAX_INLINE_SEGS];
  int32_t chunk_begin[FO_MAX_INLINE_SEGS + 1];
};

struct StepParams {
  const FoSeg* segs;           // device table (null when inline)
  const int32_t* chunk_begin;  // device table (null when inline)
  int n_seg;
  int total_chunks;
  unsigned int* status;  // optional device word where a kernel records a wait that ran out
  InlineTable inl;
};

// Walks the chunk list of one CTA: chunk c belongs to the segment s with
// chunk_begin[s] <= c < chunk_begin[s + 1]; a CTA visits chunks in increasing
// order, so the segment index only ever moves forward.
struct ChunkWalker {
  const FoSeg* segs;
  const int32_t* cb;
  int total;
  int seg, seg_begin, seg_end;
  FoSeg S;
  bool vec;

  __device__ __forceinline__ ChunkWalker(const StepParams& P)
      : segs(P.segs ? P.segs : P.inl.segs), cb(P.chunk_begin ? P.chunk_begin : P.inl.chunk_begin),
        total(P.total_chunks), seg(0) {
    seg_begin = cb[0];
    seg_end = cb[1];
    S = segs[0];
    vec = seg_vector_safe(S);
  }
  __device__ __forceinline__ void seek(int c) {
    if (c >= seg_end) {
      do { ++seg; } while (c >= cb[seg + 1]);
      S = segs[seg];
      seg_begin = cb[seg];
      seg_end = cb[seg + 1];
      vec = seg_vector_safe(S);
    }
  }
  __device__ __forceinline__ int64_t unit_base(int c, int u) const {
    return (int64_t)(c - seg_begin) * kChunk + (int64_t)(u * kThreads + threadIdx.x) * kUnit;
  }
};


// Bulk-copy staged variants (fo_step_staged.cu).  Return -1 when the combination is not
// served by a staged kernel (the caller then uses the register-path kernel).
int staged_adam_launch(const StepParams& P, const FoAdamHyper& H, int dtype, int err_bytes, int quantized,
                       int sm_count, cudaStream_t st);
int staged_momentum_launch(const StepParams& P, const FoMomentumHyper& H, int dtype, int err_bytes,
                           int state_mode, int sm_count, cudaStream_t st);

}  // namespace fo
