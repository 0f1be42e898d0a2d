// C ABI of libflashoptim_b200.so: the launch layer that the reference implements as Python
// wrappers around Triton kernels (flashoptim/optimizers.py:1535-1583 momentum, :2203-2252 Adam,
// :2446-2540 quantize / dequantize, :2835-2974 master-weight split / merge).
// Every function returns a cudaError_t value
// (0 on success) unless stated otherwise, takes raw device pointers and a CUDA
// stream handle, launches asynchronously on that stream and allocates nothing.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Element type codes.
enum FoDtype { FO_BF16 = 0, FO_FP16 = 1, FO_FP32 = 2 };

// One tensor of a multi-tensor launch.  64 bytes.
//   p     parameter, updated in place
//   g     gradient, same dtype and length as p
//   ecc   error-correction codes (int8 or int16, same length) or null
//   s0    first state: int8 codes when quantised, else param dtype; momentum /
//         exp_avg; null when the optimizer keeps no state
//   s0s   fp16 scales of s0, one per 32 elements (quantised only)
//   s1    second state (Adam exp_avg_sq): uint8 codes or param dtype
//   s1s   fp16 scales of s1
//   n     number of elements
typedef struct FoSeg {
  void* p;
  const void* g;
  void* ecc;
  void* s0;
  void* s0s;
  void* s1;
  void* s1s;
  int64_t n;
} FoSeg;

// Complements (1 - beta, 1 - weight_decay) are evaluated by the host in double
// precision: 1.0f - 0.999f is off by 1.3e-5 relative.
typedef struct FoAdamHyper {
  float lr, beta1, beta2, eps;
  float one_minus_beta1, one_minus_beta2;
  float weight_decay;  // already folded: wd*lr (decoupled) or wd (coupled)
  float decay;         // 1 - weight_decay when decoupled, else 1
  float rbc1;          // 1 / (1 - beta1^step)
  float sqrt_rbc2;     // sqrt(1 / (1 - beta2^step))
  float grad_scale;    // gradient is multiplied by this before use
  int decoupled;
} FoAdamHyper;

typedef struct FoMomentumHyper {
  float lr;
  float mom_coef;            // SGD momentum | Lion beta2
  float update_coef;         // SGD 1 - dampening | Lion beta1
  float one_minus_mom_coef;  // Lion only
  float one_minus_update_coef;  // Lion only
  float weight_decay;        // folded like FoAdamHyper.weight_decay
  float decay;               // 1 - weight_decay when decoupled or Lion, else 1
  float grad_scale;
  int lion, nesterov, decoupled;
} FoMomentumHyper;

// State storage of the momentum family.
enum FoStateMode { FO_STATE_NONE = 0, FO_STATE_Q8 = 1, FO_STATE_FULL = 2 };

enum { FO_MAX_INLINE_SEGS = 16 };

// Elements covered by one CTA iteration ("chunk").  Segment s occupies chunks
// [chunk_begin[s], chunk_begin[s+1]) with chunk_begin[s+1] - chunk_begin[s] =
// ceil(n_s / fo_chunk_elems()).
int fo_chunk_elems(void);
// Number of CTAs the step kernels are launched with on `device` (<= total chunks).
int fo_step_grid(int device);

// Kernel family of the fused steps: 1 (default) streams bf16/fp16 tensors with 8-bit
// states through shared memory with cp.async.bulk + mbarrier stages, 0 always uses the
// register-path kernels (which also serve every other combination).
void fo_set_step_variant(int variant);
int fo_get_step_variant(void);
// Grid of the staged kernels = resident CTAs x rounds (1..1024): with more than one round the
// hardware hands out the later CTAs as earlier ones finish, which evens out SMs that run at
// different paces.  A tuning knob; the built-in default is what measured best.
void fo_set_staged_rounds(int rounds);
int fo_get_staged_rounds(void);
// Optional: a zeroed device uint32 (of the current device) in which a kernel sets a bit
// when one of its bounded waits ran out (1: producer, 2: consumer of the staged kernels).
int fo_set_step_status(void* device_word);

// Multi-tensor fused steps.  `segs` / `chunk_begin` are HOST pointers when
// n_seg <= FO_MAX_INLINE_SEGS and `table_on_device` is 0 (the table then
// travels in the kernel parameters, no device memory is touched), DEVICE
// pointers otherwise.  total_chunks = chunk_begin[n_seg].
int fo_adam_step(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                 int table_on_device, int dtype, int err_bytes, int quantized, const FoAdamHyper* hyper,
                 void* stream);
int fo_momentum_step(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                     int table_on_device, int dtype, int err_bytes, int state_mode,
                     const FoMomentumHyper* hyper, void* stream);

// Group quantiser and its inverse (exact IEEE arithmetic; see ops/oracle.py).
// `x` has element type `dtype`; `q` int8 (signed) or uint8; `scales` fp16.
int fo_quantize(const void* x, int dtype, void* q, void* scales, int64_t n, int is_signed, int do_sqrt,
                int softsign, void* stream);
int fo_dequantize(const void* q, const void* scales, float* out, int64_t n, int is_signed, int do_sqrt,
                  int softsign, void* stream);

// Master-weight split: narrow (bf16/fp16) + int8/int16 codes <-> fp32 (exact).
int fo_ecc_decode(const void* narrow, int dtype, const void* ecc, int err_bytes, float* out, int64_t n,
                  void* stream);
int fo_ecc_encode(const float* x, const void* narrow, int dtype, void* ecc, int err_bytes, int64_t n,
                  void* stream);

// max |x| of a tensor, accumulated into *out (a float the caller zeroed).
int fo_maxabs(const void* x, int dtype, int64_t n, float* out, void* stream);

// ---------------------------------------------------------------------------
// Steps fused with the gradient collective over NVLink peer memory (fo_comm.cu)
// ---------------------------------------------------------------------------

enum { FO_MAX_PEERS = 8 };

// One rank's view of a group of `world` GPUs on one node.
//   grad[r]      rank r's gradient buffer (symmetric: same layout on every rank),
//                as mapped into this process; FoSeg.g is a BYTE OFFSET into it
//   multicast    NVSwitch multicast mapping of the same buffer, or null: when set,
//                full aligned units are fetched with multimem.ld_reduce
//   pad[r]       rank r's signal pad: uint32 words [channel * FO_MAX_PEERS + src]
//   status       4 local uint32 words, zeroed by the host before first use:
//                [0] bit mask of channels whose wait timed out, [1] 1 + rank that
//                was missing, [2] CTA counter of the step / reduce kernels, [3] CTA counter
//                of the all-gather kernel (internal; the two families may overlap in time)
//   epoch        value published / awaited on the channels; grows by one per use
//   ready_channel  flag "my buffer holds this epoch's gradients"
//   done_channel   flag "I have finished reading everybody's buffer for this epoch"
//   grad_out     optional: the averaged gradient is also written to
//                grad_out + (FoSeg.g + unit offset - grad_out_sub)
//   timeout_ns   limit of every device-side wait
//   max_ctas     cap on the number of CTAs, so that a link-bound kernel running beside
//                backward leaves the SMs to the GEMMs
//   push         step kernels only, optional "all-gather on write": every updated parameter
//                unit is also stored, in the parameter dtype, at byte offset
//                (FoSeg.g + unit offset + param_out_delta) of param_out[r] for every rank r
//                (or once through the multicast mapping param_out_mc), and the kernel then
//                publishes push_epoch on pushed_channel.  A rank that waits for all ranks'
//                pushed flags holds every rank's fresh parameters without an all-gather.
//   variant      step kernels: 1 selects the bulk-copy staged kernels (a producer thread streams
//                the ranks' gradient chunks and the local state through shared memory with
//                cp.async.bulk; few CTAs saturate NVLink) for bf16 / fp16 parameters with 8-bit
//                states and peer loads (multicast null); every other case, and 0, runs the
//                register-path kernels
typedef struct FoCommArgs {
  const void* grad[FO_MAX_PEERS];
  const void* multicast;
  uint32_t* pad[FO_MAX_PEERS];
  uint32_t* status;
  void* grad_out;
  int64_t grad_out_sub;
  uint64_t timeout_ns;
  uint32_t epoch;
  int world, rank;
  int ready_channel, done_channel;
  int max_ctas;  // upper bound on the launch grid (0: fill the GPU); NVLink-bound work needs few SMs
  int push;      // 0: no parameter push (the fields below are ignored)
  void* param_out[FO_MAX_PEERS];
  void* param_out_mc;
  int64_t param_out_delta;
  uint32_t push_epoch;
  int pushed_channel;
  int variant;  // step kernels: 0 register path; 1 bulk-copy staged kernels where they apply
  int flags;    // FO_COMM_* bits
} FoCommArgs;

// FoCommArgs.flags, for callers that move the bytes themselves (copy engines) and use the
// step kernels only for the arithmetic:
//   NO_BARRIER   the kernel neither publishes "ready" nor waits for it
//   NO_SIGNAL    the kernel publishes neither "done" nor "pushed"
//   PUSH_LOCAL   the parameter push stores into param_out[rank] only
enum { FO_COMM_NO_BARRIER = 1, FO_COMM_NO_SIGNAL = 2, FO_COMM_PUSH_LOCAL = 4 };

// Elements per CTA iteration ("chunk", for the chunk prefix) of the kernel that
// fo_adam_step_peer / fo_momentum_step_peer will run for these arguments; `q8_states` is
// `quantized` of the Adam call, or state_mode == FO_STATE_Q8 of the momentum call.  Register
// path with peer loads: the fewer ranks, the more units a thread keeps in flight; with
// multimem always four units; staged kernels: one unit.
int fo_comm_step_chunk_elems(const FoCommArgs* comm, int dtype, int q8_states);

// `segs` and `chunk_begin` are DEVICE pointers.  The gradient of every element
// is hyper->grad_scale times the sum over ranks (pass 1 / world for a mean).
int fo_adam_step_peer(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks, int dtype,
                      int err_bytes, int quantized, const FoAdamHyper* hyper, const FoCommArgs* comm,
                      void* stream);
int fo_momentum_step_peer(const FoSeg* segs, const int32_t* chunk_begin, int n_seg, int total_chunks,
                          int dtype, int err_bytes, int state_mode, const FoMomentumHyper* hyper,
                          const FoCommArgs* comm, void* stream);
// out[i] = scale * sum_r grad[r][src_offset_bytes + i] for n elements (no update).
int fo_reduce_peer(int64_t n, int64_t src_offset_bytes, void* out, int dtype, float scale,
                   const FoCommArgs* comm, void* stream);
// First shot of a two-shot all-reduce: rank r averages slice r (of `world` slices) of the n
// elements at src_offset_bytes of every rank's buffer and stores it at dst_offset_bytes of
// EVERY rank's buffer.  Once all ranks have published done(epoch), each buffer holds the full
// averaged vector at dst_offset_bytes.
int fo_reduce_bcast_peer(int64_t n, int64_t src_offset_bytes, int64_t dst_offset_bytes, int dtype,
                         float scale, const FoCommArgs* comm, void* stream);
// All-gather inside the symmetric buffer: every rank pulls slot s (slot_bytes
// each, a multiple of 16) from rank s into its own copy.
int fo_allgather_peer(int64_t slot_bytes, const FoCommArgs* comm, void* stream);
// Publish / await comm->epoch on one channel from a one-CTA kernel.
int fo_comm_signal(const FoCommArgs* comm, int channel, void* stream);
int fo_comm_wait(const FoCommArgs* comm, int channel, void* stream);
// One-CTA kernel: publish comm->epoch on the ready channel, then await every rank's.
int fo_comm_barrier(const FoCommArgs* comm, void* stream);
// cudaMemcpyAsync(device to device) on `stream`: between two mappings of symmetric buffers the
// driver moves the bytes over NVLink with a copy engine, no SM involved.
int fo_memcpy_async(void* dst, const void* src, int64_t nbytes, void* stream);

// ---------------------------------------------------------------------------
// Test support (fo_probe.cu): the fast forms of the master-weight split that the step kernels
// inline, applied to caller-supplied fp32 values.  n a multiple of 8, pointers 16-byte aligned.
// ---------------------------------------------------------------------------
int fo_probe_fast_ecc_split(const float* x, int dtype, int err_bytes, void* narrow, void* ecc, int64_t n,
                            void* stream);
int fo_probe_fast_ecc_merge(const void* narrow, int dtype, const void* ecc, int err_bytes, float* out, int64_t n,
                            void* stream);

#ifdef __cplusplus
}
#endif
