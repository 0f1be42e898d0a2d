// Stand-alone group quantiser / dequantiser, master-weight split and maxabs.
//
// These run at state creation, checkpoint save/load and fp32 export/import, so
// they use exact IEEE arithmetic (explicit round-to-nearest intrinsics, which
// the compiler never contracts into FMAs) and reproduce the PyTorch formulation
// in ops/oracle.py bit for bit.  What they compute matches
// flashoptim/optimizers.py:2610-2676 (quantise), :2541-2607 (dequantise),
// :2726-2776 (error-correction encode / decode).
#include <type_traits>

#include "fo_api.h"
#include "fo_common.cuh"

namespace fo {

constexpr int kQThreads = 256;

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, int64_t i) {
  if constexpr (sizeof(T) == 4) return p[i];
  else if constexpr (std::is_same<T, __half>::value) return __half2float(p[i]);
  else return __bfloat162float(p[i]);
}

// One thread per unit of 8 elements; four lanes form a group.
template <typename T, bool kSigned, bool kSqrt, bool kSoftsign>
__global__ void __launch_bounds__(kQThreads) quantize_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                             __half* __restrict__ scales, int64_t n) {
  const int64_t n_units = ((n + kGroup - 1) / kGroup) * (kGroup / kUnit);
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit - threadIdx.x < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    const int64_t base = unit * kUnit;
    float v[kUnit];
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      float e = (unit < n_units && base + i < n) ? load_as_float(x, base + i) : 0.0f;
      if (kSqrt) e = __fsqrt_rn(e);
      v[i] = e;
      a = fmaxf(a, fabsf(e));
    }
    a = fmaxf(group_max(a), 1e-12f);
    const float qmax = kSigned ? 127.0f : 255.0f;
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      float t = __fdiv_rn(v[i], a);
      if (kSoftsign) t = __fdiv_rn(__fmul_rn(t, 2.0f), __fadd_rn(fabsf(t), 1.0f));
      const float r = floorf(__fadd_rn(__fmul_rn(t, qmax), 0.5f));
      if (unit < n_units && base + i < n) q[base + i] = kSigned ? (uint8_t)(int8_t)(int)r : (uint8_t)(int)r;
    }
    if ((threadIdx.x & 3) == 0 && unit < n_units && base < n) scales[base >> 5] = __float2half_rn(a);
  }
}

template <bool kSigned, bool kSqrt, bool kSoftsign>
__global__ void __launch_bounds__(kQThreads) dequantize_kernel(const uint8_t* __restrict__ q,
                                                               const __half* __restrict__ scales,
                                                               float* __restrict__ out, int64_t n) {
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    const int64_t base = unit * kUnit;
    const float sc = __half2float(scales[base >> 5]);
    const float qmax = kSigned ? 127.0f : 255.0f;
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      if (base + i < n) {
        const float c = kSigned ? (float)(int8_t)q[base + i] : (float)q[base + i];
        float t = __fdiv_rn(c, qmax);
        if (kSoftsign) t = __fdiv_rn(t, __fsub_rn(2.0f, fabsf(t)));
        float r = __fmul_rn(t, sc);
        if (kSqrt) r = __fmul_rn(r, r);
        out[base + i] = r;
      }
    }
  }
}

// Exact 2^e for e in [-126, 127].
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((e + 127) << 23); }

template <typename T>
__device__ __forceinline__ int ecc_log_scale(T w) {
  constexpr int M = Elem<T>::kMant;
  constexpr int bias = std::is_same<T, __half>::value ? 15 : 127;
  uint16_t bits;
  if constexpr (std::is_same<T, __half>::value) bits = __half_as_ushort(w);
  else bits = __bfloat16_as_ushort(w);
  const int field = (bits & 0x7FFF) >> M;
  const int e = field == 0 ? 1 - bias : field - bias;
  return e - M - 1;
}

template <typename T, typename E>
__global__ void __launch_bounds__(kQThreads) ecc_decode_kernel(const T* __restrict__ w, const E* __restrict__ ecc,
                                                               float* __restrict__ out, int64_t n) {
  const float smax = sizeof(E) == 1 ? 127.0f : 32767.0f;
  for (int64_t i = (int64_t)blockIdx.x * kQThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kQThreads) {
    const T wn = w[i];
    const int ls = ecc_log_scale(wn);
    const int h = ls >> 1;  // floor(ls / 2)
    const float corr = __fdiv_rn((float)ecc[i], smax);
    const float e = __fmul_rn(__fmul_rn(corr, pow2i(h)), pow2i(ls - h));
    out[i] = __fadd_rn(load_as_float(w, i), e);
  }
}

template <typename T, typename E>
__global__ void __launch_bounds__(kQThreads) ecc_encode_kernel(const float* __restrict__ x, const T* __restrict__ w,
                                                               E* __restrict__ ecc, int64_t n) {
  const float smax = sizeof(E) == 1 ? 127.0f : 32767.0f;
  for (int64_t i = (int64_t)blockIdx.x * kQThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kQThreads) {
    const T wn = w[i];
    const int neg = -ecc_log_scale(wn);
    const int h = neg >> 1;
    const float e = __fsub_rn(x[i], load_as_float(w, i));
    float en = __fmul_rn(__fmul_rn(e, pow2i(h)), pow2i(neg - h));
    en = fminf(fmaxf(en, -1.0f), 1.0f);
    const float s = __fmul_rn(en, smax);
    const float r = copysignf(floorf(__fadd_rn(fabsf(s), 0.5f)), s);
    ecc[i] = (E)(int)r;
  }
}

template <typename T>
__global__ void __launch_bounds__(kQThreads) maxabs_kernel(const T* __restrict__ x, int64_t n, float* out) {
  float a = 0.0f;
  for (int64_t i = (int64_t)blockIdx.x * kQThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kQThreads)
    a = fmaxf(a, fabsf(load_as_float(x, i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(kFullMask, a, o));
  // non-negative floats order like their bit patterns; NaN inputs are dropped by fmaxf
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(a));
}

static int blocks_for(int64_t work_items) {
  int64_t b = (work_items + kQThreads - 1) / kQThreads;
  const int64_t cap = 148 * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

template <typename T, bool kSigned, bool kSqrt>
static void launch_quant(const void* x, void* q, void* scales, int64_t n, int softsign, cudaStream_t st) {
  const int64_t n_units = ((n + kGroup - 1) / kGroup) * (kGroup / kUnit);
  const int grid = blocks_for(n_units);
  if (softsign)
    quantize_kernel<T, kSigned, kSqrt, true><<<grid, kQThreads, 0, st>>>((const T*)x, (uint8_t*)q, (__half*)scales, n);
  else
    quantize_kernel<T, kSigned, kSqrt, false><<<grid, kQThreads, 0, st>>>((const T*)x, (uint8_t*)q, (__half*)scales, n);
}
template <typename T>
static void launch_quant_t(const void* x, void* q, void* scales, int64_t n, int is_signed, int do_sqrt,
                           int softsign, cudaStream_t st) {
  if (is_signed) {
    if (do_sqrt) launch_quant<T, true, true>(x, q, scales, n, softsign, st);
    else launch_quant<T, true, false>(x, q, scales, n, softsign, st);
  } else {
    if (do_sqrt) launch_quant<T, false, true>(x, q, scales, n, softsign, st);
    else launch_quant<T, false, false>(x, q, scales, n, softsign, st);
  }
}

template <bool kSigned, bool kSqrt>
static void launch_dequant(const void* q, const void* scales, float* out, int64_t n, int softsign,
                           cudaStream_t st) {
  const int grid = blocks_for((n + kUnit - 1) / kUnit);
  if (softsign)
    dequantize_kernel<kSigned, kSqrt, true><<<grid, kQThreads, 0, st>>>((const uint8_t*)q, (const __half*)scales, out, n);
  else
    dequantize_kernel<kSigned, kSqrt, false><<<grid, kQThreads, 0, st>>>((const uint8_t*)q, (const __half*)scales, out, n);
}

}  // namespace fo

extern "C" int fo_quantize(const void* x, int dtype, void* q, void* scales, int64_t n, int is_signed,
                           int do_sqrt, int softsign, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FO_BF16: fo::launch_quant_t<__nv_bfloat16>(x, q, scales, n, is_signed, do_sqrt, softsign, st); break;
    case FO_FP16: fo::launch_quant_t<__half>(x, q, scales, n, is_signed, do_sqrt, softsign, st); break;
    case FO_FP32: fo::launch_quant_t<float>(x, q, scales, n, is_signed, do_sqrt, softsign, st); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}

extern "C" int fo_dequantize(const void* q, const void* scales, float* out, int64_t n, int is_signed,
                             int do_sqrt, int softsign, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (is_signed) {
    if (do_sqrt) fo::launch_dequant<true, true>(q, scales, out, n, softsign, st);
    else fo::launch_dequant<true, false>(q, scales, out, n, softsign, st);
  } else {
    if (do_sqrt) fo::launch_dequant<false, true>(q, scales, out, n, softsign, st);
    else fo::launch_dequant<false, false>(q, scales, out, n, softsign, st);
  }
  return (int)cudaGetLastError();
}

extern "C" int fo_ecc_decode(const void* narrow, int dtype, const void* ecc, int err_bytes, float* out,
                             int64_t n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = fo::blocks_for(n);
  if (dtype == FO_BF16 && err_bytes == 1)
    fo::ecc_decode_kernel<<<grid, fo::kQThreads, 0, st>>>((const __nv_bfloat16*)narrow, (const int8_t*)ecc, out, n);
  else if (dtype == FO_BF16 && err_bytes == 2)
    fo::ecc_decode_kernel<<<grid, fo::kQThreads, 0, st>>>((const __nv_bfloat16*)narrow, (const int16_t*)ecc, out, n);
  else if (dtype == FO_FP16 && err_bytes == 1)
    fo::ecc_decode_kernel<<<grid, fo::kQThreads, 0, st>>>((const __half*)narrow, (const int8_t*)ecc, out, n);
  else if (dtype == FO_FP16 && err_bytes == 2)
    fo::ecc_decode_kernel<<<grid, fo::kQThreads, 0, st>>>((const __half*)narrow, (const int16_t*)ecc, out, n);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int fo_ecc_encode(const float* x, const void* narrow, int dtype, void* ecc, int err_bytes,
                             int64_t n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = fo::blocks_for(n);
  if (dtype == FO_BF16 && err_bytes == 1)
    fo::ecc_encode_kernel<<<grid, fo::kQThreads, 0, st>>>(x, (const __nv_bfloat16*)narrow, (int8_t*)ecc, n);
  else if (dtype == FO_BF16 && err_bytes == 2)
    fo::ecc_encode_kernel<<<grid, fo::kQThreads, 0, st>>>(x, (const __nv_bfloat16*)narrow, (int16_t*)ecc, n);
  else if (dtype == FO_FP16 && err_bytes == 1)
    fo::ecc_encode_kernel<<<grid, fo::kQThreads, 0, st>>>(x, (const __half*)narrow, (int8_t*)ecc, n);
  else if (dtype == FO_FP16 && err_bytes == 2)
    fo::ecc_encode_kernel<<<grid, fo::kQThreads, 0, st>>>(x, (const __half*)narrow, (int16_t*)ecc, n);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int fo_maxabs(const void* x, int dtype, int64_t n, float* out, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = fo::blocks_for((n + 7) / 8);
  switch (dtype) {
    case FO_BF16: fo::maxabs_kernel<<<grid, fo::kQThreads, 0, st>>>((const __nv_bfloat16*)x, n, out); break;
    case FO_FP16: fo::maxabs_kernel<<<grid, fo::kQThreads, 0, st>>>((const __half*)x, n, out); break;
    case FO_FP32: fo::maxabs_kernel<<<grid, fo::kQThreads, 0, st>>>((const float*)x, n, out); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}
