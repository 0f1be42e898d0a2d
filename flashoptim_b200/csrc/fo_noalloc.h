// Allocation-free multi-tensor Adam/AdamW step.
//
// This entry point has no counterpart in the reference (which is Python and
// leaves every allocation to PyTorch).  It exists for callers that must not
// allocate device memory at the moment they step the optimizer:
//   * a gradient hook that fires in the middle of backward on a side stream --
//     cudaMalloc / cudaFree synchronise the whole device, so an allocation
//     there stalls the backward kernels that the step is meant to overlap;
//   * a C/C++ host program that has already handed all device memory to its own
//     pool (or to another framework's caching allocator) and has no allocator
//     of this library's to call.
// fo_adam_step() serves long tensor lists from a device-resident segment table
// that its caller has to allocate and fill.  Here that table lives in a
// file-scope __device__ array inside the library instead, so the caller passes
// only its own tensors, described by a HOST array of segments.
//
// Limits and rules:
//   * at most FO_NOALLOC_MAX_SEGS tensors per call and fewer than 2^31 chunks
//     (2048 elements each) in total; larger requests are refused with
//     FO_NOALLOC_ERR_TOO_MANY_SEGS / FO_NOALLOC_ERR_TOO_MANY_ELEMS and a message
//     on stderr, nothing is launched;
//   * the table costs FO_NOALLOC_MAX_SEGS * 64 + (FO_NOALLOC_MAX_SEGS + 1) * 4
//     bytes (about 136 KB) of device memory on every GPU that loads the
//     library, from load until the process exits;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and caches it; make
//     that first call before starting any stream capture;
//   * all calls on a device share the one table.  Each call rewrites the part
//     it uses before launching (stale entries beyond n_seg are never read, so
//     nothing needs clearing); the kernels that write the table and the step
//     kernel are ordered on `stream`.  Two calls whose work overlaps on the
//     GPU (different streams, no event between them) race on the table:
//     serialise them.
//   * no cudaMalloc, cudaFree, cudaMemcpy or other allocating or synchronising
//     call is made.  The segments reach the device inside the launch
//     parameters of small table-writing kernels (48 segments per launch), so
//     `segs` may be any host memory, pageable or pinned, is read completely
//     before the call returns and may be reused at once, and the host never
//     waits for `stream`.
//   * every argument is validated before the first launch: a refused call has
//     touched neither the table nor the stream.
#pragma once

#include "fo_api.h"

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FO_NOALLOC_MAX_SEGS = 2048,
  FO_NOALLOC_ERR_TOO_MANY_SEGS = -1,
  FO_NOALLOC_ERR_TOO_MANY_ELEMS = -2,
  FO_NOALLOC_ERR_BAD_ARGUMENT = -3
};

// One fused Adam/AdamW step over `n_seg` tensors, same arithmetic and the same
// meaning of `dtype`, `err_bytes`, `quantized` and `hyper` as fo_adam_step().
// Returns 0, one of the negative FO_NOALLOC_ERR_* codes, or a positive
// cudaError_t value.
int fo_adam_step_noalloc(const FoSeg* segs, int n_seg, int dtype, int err_bytes, int quantized,
                         const FoAdamHyper* hyper, void* stream);

#ifdef __cplusplus
}
#endif
