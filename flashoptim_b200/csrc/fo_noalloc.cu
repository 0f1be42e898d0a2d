// Allocation-free variant of the multi-tensor Adam step: its segment table is a
// file-scope __device__ array of this library instead of caller-allocated
// device memory.  See fo_noalloc.h for who needs this and the rules of use.
#include <stdio.h>

#include "fo_noalloc.h"
#include "fo_step_core.cuh"

namespace fo {
namespace {

constexpr int kNaThreads = 256;
constexpr int kNaChunk = kNaThreads * kUnit;  // one unit per thread per chunk
constexpr int kNaCtasPerSm = 4;
constexpr int kMaxDevices = 64;

struct NoallocTable {
  FoSeg segs[FO_NOALLOC_MAX_SEGS];
  int32_t chunk_begin[FO_NOALLOC_MAX_SEGS + 1];
};

// The scratch itself.  In host code this name is only a handle for
// cudaGetSymbolAddress; the address a kernel can use is looked up per device.
static __device__ __align__(256) unsigned char g_noalloc_table[sizeof(NoallocTable)];

template <typename T, int kErr, bool kQ>
__global__ void __launch_bounds__(kNaThreads, kNaCtasPerSm)
    adam_noalloc_kernel(const NoallocTable* __restrict__ table, int total_chunks,
                        const __grid_constant__ FoAdamHyper H) {
  using Regs = UnitRegs<T, kErr, 2, kQ>;
  const int32_t* cb = table->chunk_begin;
  int seg = 0;
  int seg_begin = cb[0], seg_end = cb[1];
  FoSeg S = table->segs[0];
  bool vec = seg_vector_safe(S);
  for (int c = blockIdx.x; c < total_chunks; c += gridDim.x) {
    if (c >= seg_end) {
      do { ++seg; } while (c >= cb[seg + 1]);
      S = table->segs[seg];
      seg_begin = cb[seg];
      seg_end = cb[seg + 1];
      vec = seg_vector_safe(S);
    }
    const int64_t base = (int64_t)(c - seg_begin) * kNaChunk + (int64_t)threadIdx.x * kUnit;
    Regs r;
    load_unit_state(r, S, base, vec);
    load_unit_grad(r, S, base, vec);
    float2 p[4], g[4], m[4], v[4];
    unpack8<T>(r.g, g);
    widen_unit(r, p, m, v);
    adam_update8<kQ>(p, g, m, v, H);
    store_unit(r, S, base, vec, p, m, v);
  }
}

// The table is written by small kernels that carry the segments in their launch parameters:
// the driver copies launch parameters when the launch is issued, so the caller's `segs`
// array is free again when fo_adam_step_noalloc() returns, whatever kind of host memory it
// is, and the host never waits for the stream (a cudaMemcpyAsync from pageable memory would
// make it wait, from pinned memory it would read `segs` later).
constexpr int kFillSegs = 48;  // 48 * 64 + 49 * 4 + 8 bytes: below the 4 KB of launch parameters
struct FillArgs {
  FoSeg segs[kFillSegs];
  int32_t chunk_begin[kFillSegs + 1];  // chunk_begin[first .. first + count]
  int first, count;
};
__global__ void fill_table_kernel(NoallocTable* table, const __grid_constant__ FillArgs a) {
  for (int i = threadIdx.x; i < a.count; i += blockDim.x) table->segs[a.first + i] = a.segs[i];
  for (int i = threadIdx.x; i <= a.count; i += blockDim.x) table->chunk_begin[a.first + i] = a.chunk_begin[i];
}

// Device address of g_noalloc_table on each device, filled on first use.
NoallocTable* g_table_addr[kMaxDevices];
int g_sm_count[kMaxDevices];

int table_for_current_device(NoallocTable** out, int* sms) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (g_table_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_table);
    if (e != cudaSuccess) return (int)e;
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    g_sm_count[dev] = n > 0 ? n : 148;
    g_table_addr[dev] = static_cast<NoallocTable*>(ptr);
  }
  *out = g_table_addr[dev];
  *sms = g_sm_count[dev];
  return 0;
}

template <typename T, int kErr>
int launch_q(const NoallocTable* t, int total, const FoAdamHyper& H, int quantized, int grid, cudaStream_t st) {
  if (quantized) adam_noalloc_kernel<T, kErr, true><<<grid, kNaThreads, 0, st>>>(t, total, H);
  else adam_noalloc_kernel<T, kErr, false><<<grid, kNaThreads, 0, st>>>(t, total, H);
  return (int)cudaGetLastError();
}
template <typename T>
int launch_e(const NoallocTable* t, int total, const FoAdamHyper& H, int err, int quantized, int grid,
             cudaStream_t st) {
  if constexpr (Elem<T>::kNarrow) {
    if (err == 1) return launch_q<T, 1>(t, total, H, quantized, grid, st);
    if (err == 2) return launch_q<T, 2>(t, total, H, quantized, grid, st);
  }
  if (err != 0) return FO_NOALLOC_ERR_BAD_ARGUMENT;
  return launch_q<T, 0>(t, total, H, quantized, grid, st);
}

}  // namespace
}  // namespace fo

extern "C" int fo_adam_step_noalloc(const FoSeg* segs, int n_seg, int dtype, int err_bytes, int quantized,
                                    const FoAdamHyper* hyper, void* stream) {
  using namespace fo;
  if (segs == nullptr || hyper == nullptr || n_seg < 0) {
    fprintf(stderr, "fo_adam_step_noalloc: null argument or negative segment count\n");
    return FO_NOALLOC_ERR_BAD_ARGUMENT;
  }
  if (dtype != FO_BF16 && dtype != FO_FP16 && dtype != FO_FP32) {
    fprintf(stderr, "fo_adam_step_noalloc: unknown dtype code %d\n", dtype);
    return FO_NOALLOC_ERR_BAD_ARGUMENT;
  }
  if (err_bytes < 0 || err_bytes > 2 || (dtype == FO_FP32 && err_bytes != 0)) {
    fprintf(stderr, "fo_adam_step_noalloc: err_bytes %d is not valid for dtype code %d\n", err_bytes, dtype);
    return FO_NOALLOC_ERR_BAD_ARGUMENT;
  }
  if (n_seg == 0) return 0;
  if (n_seg > FO_NOALLOC_MAX_SEGS) {
    fprintf(stderr, "fo_adam_step_noalloc: %d tensors exceed the built-in table of %d; split the call\n",
            n_seg, (int)FO_NOALLOC_MAX_SEGS);
    return FO_NOALLOC_ERR_TOO_MANY_SEGS;
  }
  // chunk prefix on the host; 8 KB of stack.  Everything is validated before the first launch.
  int32_t chunk_begin[FO_NOALLOC_MAX_SEGS + 1];
  int64_t total = 0;
  chunk_begin[0] = 0;
  for (int i = 0; i < n_seg; ++i) {
    if (segs[i].n < 0) {
      fprintf(stderr, "fo_adam_step_noalloc: segment %d has a negative length\n", i);
      return FO_NOALLOC_ERR_BAD_ARGUMENT;
    }
    total += (segs[i].n + kNaChunk - 1) / kNaChunk;
    if (total >= (int64_t(1) << 31)) {
      fprintf(stderr, "fo_adam_step_noalloc: more than 2^31 chunks of %d elements; split the call\n", kNaChunk);
      return FO_NOALLOC_ERR_TOO_MANY_ELEMS;
    }
    chunk_begin[i + 1] = (int32_t)total;
  }
  if (total == 0) return 0;

  NoallocTable* table = nullptr;
  int sms = 0;
  int rc = table_for_current_device(&table, &sms);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  for (int first = 0; first < n_seg; first += kFillSegs) {
    FillArgs a;
    a.first = first;
    a.count = n_seg - first < kFillSegs ? n_seg - first : kFillSegs;
    for (int i = 0; i < a.count; ++i) a.segs[i] = segs[first + i];
    for (int i = 0; i <= a.count; ++i) a.chunk_begin[i] = chunk_begin[first + i];
    fill_table_kernel<<<1, 64, 0, st>>>(table, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  int grid = sms * kNaCtasPerSm;
  if (total < grid) grid = (int)total;
  switch (dtype) {
    case FO_BF16: return launch_e<__nv_bfloat16>(table, (int)total, *hyper, err_bytes, quantized, grid, st);
    case FO_FP16: return launch_e<__half>(table, (int)total, *hyper, err_bytes, quantized, grid, st);
  }
  return launch_e<float>(table, (int)total, *hyper, err_bytes, quantized, grid, st);
}
