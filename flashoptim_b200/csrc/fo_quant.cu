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

// Every kernel here gives a thread one unit of 8 consecutive elements per iteration and moves
// it with 16-byte (8-byte for byte-sized elements) vector accesses when the tensor's base
// address allows and the unit is whole; tails and unaligned tensors go element by element.
// The arithmetic per element is the same in both paths.

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, int64_t i) {
  if constexpr (sizeof(T) == 4) return p[i];
  else if constexpr (std::is_same<T, __half>::value) return __half2float(p[i]);
  else return __bfloat162float(p[i]);
}

template <typename T>
__device__ __forceinline__ bool aligned_for_units(const T* p) {
  constexpr uintptr_t need = sizeof(T) * kUnit >= 16 ? 16 : sizeof(T) * kUnit;
  return (reinterpret_cast<uintptr_t>(p) & (need - 1)) == 0;
}

// 8 elements of any supported float type -> fp32 (exact widening); zero beyond n.
template <typename T>
__device__ __forceinline__ void load8f(const T* p, int64_t base, int64_t n, bool vec, float (&v)[kUnit]) {
  if (vec && base + kUnit <= n) {
    if constexpr (sizeof(T) == 4) {
      const uint4 a = ld16_stream(p + base), b = ld16_stream(p + base + 4);
      v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
      v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
    } else {
      const uint4 a = ld16_stream(p + base);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if constexpr (std::is_same<T, __half>::value) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
          v[2 * i] = f.x;
          v[2 * i + 1] = f.y;
        } else {
          v[2 * i] = __uint_as_float(w[i] << 16);
          v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i) v[i] = base + i < n ? load_as_float(p, base + i) : 0.0f;
  }
}
// 8 narrow elements, raw 16-bit patterns (for the exponent arithmetic of the correction).
template <typename T>
__device__ __forceinline__ void load8bits(const T* p, int64_t base, int64_t n, bool vec, uint16_t (&h)[kUnit]) {
  static_assert(sizeof(T) == 2, "narrow types only");
  if (vec && base + kUnit <= n) {
    const uint4 a = ld16_stream(p + base);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      h[2 * i] = (uint16_t)(w[i] & 0xffffu);
      h[2 * i + 1] = (uint16_t)(w[i] >> 16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i) h[i] = base + i < n ? reinterpret_cast<const uint16_t*>(p)[base + i] : (uint16_t)0;
  }
}
__device__ __forceinline__ void store8f(float* p, int64_t base, int64_t n, bool vec, const float (&v)[kUnit]) {
  if (vec && base + kUnit <= n) {
    st16(p + base, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
    st16(p + base + 4,
         make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i)
      if (base + i < n) p[base + i] = v[i];
  }
}
// 8 one-byte or two-byte integers (two's complement in the low bits of c[i]).
template <typename E>
__device__ __forceinline__ void store8i(E* p, int64_t base, int64_t n, bool vec, const int (&c)[kUnit]) {
  if (vec && base + kUnit <= n) {
    if constexpr (sizeof(E) == 1) {
      uint2 o;
      o.x = (c[0] & 0xff) | ((c[1] & 0xff) << 8) | ((c[2] & 0xff) << 16) | ((uint32_t)(c[3] & 0xff) << 24);
      o.y = (c[4] & 0xff) | ((c[5] & 0xff) << 8) | ((c[6] & 0xff) << 16) | ((uint32_t)(c[7] & 0xff) << 24);
      st8(p + base, o);
    } else {
      uint4 o;
      o.x = (c[0] & 0xffff) | ((uint32_t)(c[1] & 0xffff) << 16);
      o.y = (c[2] & 0xffff) | ((uint32_t)(c[3] & 0xffff) << 16);
      o.z = (c[4] & 0xffff) | ((uint32_t)(c[5] & 0xffff) << 16);
      o.w = (c[6] & 0xffff) | ((uint32_t)(c[7] & 0xffff) << 16);
      st16(p + base, o);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i)
      if (base + i < n) p[base + i] = (E)c[i];
  }
}
template <typename E>
__device__ __forceinline__ void load8i(const E* p, int64_t base, int64_t n, bool vec, int (&c)[kUnit]) {
  if (vec && base + kUnit <= n) {
    if constexpr (sizeof(E) == 1) {
      const uint2 a = ld8_stream(p + base);
      const uint32_t w[2] = {a.x, a.y};
#pragma unroll
      for (int i = 0; i < kUnit; ++i) {
        const uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
        c[i] = std::is_signed<E>::value ? (int)(int8_t)b : (int)b;
      }
    } else {
      const uint4 a = ld16_stream(p + base);
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int i = 0; i < kUnit; ++i) c[i] = (int)(int16_t)((w[i >> 1] >> (16 * (i & 1))) & 0xffffu);
    }
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i) c[i] = base + i < n ? (int)p[base + i] : 0;
  }
}

// One thread per unit of 8 elements; four lanes form a group.
template <typename T, bool kSigned, bool kSqrt, bool kSoftsign>
__global__ void __launch_bounds__(kQThreads) quantize_kernel(const T* __restrict__ x, uint8_t* __restrict__ q,
                                                             __half* __restrict__ scales, int64_t n) {
  const int64_t n_units = ((n + kGroup - 1) / kGroup) * (kGroup / kUnit);
  const bool vec = aligned_for_units(x) && aligned_for_units(q);
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit - threadIdx.x < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    const int64_t base = unit * kUnit;
    const bool live = unit < n_units;
    float v[kUnit];
    load8f(x, base, live ? n : 0, vec, v);  // zero beyond the tensor: padding cannot raise the absmax
    float a = 0.0f;
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      if (kSqrt) v[i] = __fsqrt_rn(v[i]);
      a = fmaxf(a, fabsf(v[i]));
    }
    a = fmaxf(group_max(a), 1e-12f);
    const float qmax = kSigned ? 127.0f : 255.0f;
    int c[kUnit];
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      float t = __fdiv_rn(v[i], a);
      if (kSoftsign) t = __fdiv_rn(__fmul_rn(t, 2.0f), __fadd_rn(fabsf(t), 1.0f));
      c[i] = (int)floorf(__fadd_rn(__fmul_rn(t, qmax), 0.5f));
    }
    if (live) {
      if (kSigned) store8i(reinterpret_cast<int8_t*>(q), base, n, vec, c);
      else store8i(q, base, n, vec, c);
    }
    if ((threadIdx.x & 3) == 0 && live && base < n) scales[base >> 5] = __float2half_rn(a);
  }
}

template <bool kSigned, bool kSqrt, bool kSoftsign>
__global__ void __launch_bounds__(kQThreads) dequantize_kernel(const uint8_t* __restrict__ q,
                                                               const __half* __restrict__ scales,
                                                               float* __restrict__ out, int64_t n) {
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  const bool vec = aligned_for_units(q) && aligned_for_units(out);
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    const int64_t base = unit * kUnit;
    const float sc = __half2float(scales[base >> 5]);
    const float qmax = kSigned ? 127.0f : 255.0f;
    int c[kUnit];
    if (kSigned) load8i(reinterpret_cast<const int8_t*>(q), base, n, vec, c);
    else load8i(q, base, n, vec, c);
    float r[kUnit];
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      float t = __fdiv_rn((float)c[i], qmax);
      if (kSoftsign) t = __fdiv_rn(t, __fsub_rn(2.0f, fabsf(t)));
      r[i] = __fmul_rn(t, sc);
      if (kSqrt) r[i] = __fmul_rn(r[i], r[i]);
    }
    store8f(out, base, n, vec, r);
  }
}

// Exact 2^e for e in [-126, 127].
__device__ __forceinline__ float pow2i(int e) { return __int_as_float((e + 127) << 23); }

// c / smax, correctly rounded, for an integer code |c| <= smax in {127, 32767}: the rounded
// reciprocal, one product and one FMA-corrected refinement.  Equal to IEEE division for every
// code (checked exhaustively against fp32 division; tests/test_kernels_gpu.py compares the
// kernel with the PyTorch formulation over all codes) at a third of its instructions.
__device__ __forceinline__ float div_by_code_range(float c, float smax) {
  const float r = smax == 127.0f ? (1.0f / 127.0f) : (1.0f / 32767.0f);
  const float q0 = __fmul_rn(c, r);
  const float rem = __fmaf_rn(-q0, smax, c);
  return __fmaf_rn(rem, r, q0);
}

template <typename T>
__device__ __forceinline__ int ecc_log_scale_bits(uint16_t bits) {
  constexpr int M = Elem<T>::kMant;
  constexpr int bias = std::is_same<T, __half>::value ? 15 : 127;
  const int field = (bits & 0x7FFF) >> M;
  const int e = field == 0 ? 1 - bias : field - bias;
  return e - M - 1;
}
template <typename T>
__device__ __forceinline__ float narrow_bits_to_float(uint16_t bits) {
  if constexpr (std::is_same<T, __half>::value) return __half2float(__ushort_as_half(bits));
  else return __uint_as_float((uint32_t)bits << 16);
}

template <typename T, typename E>
__global__ void __launch_bounds__(kQThreads) ecc_decode_kernel(const T* __restrict__ w, const E* __restrict__ ecc,
                                                               float* __restrict__ out, int64_t n) {
  const float smax = sizeof(E) == 1 ? 127.0f : 32767.0f;
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  const bool vec = aligned_for_units(w) && aligned_for_units(ecc) && aligned_for_units(out);
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    const int64_t base = unit * kUnit;
    uint16_t h[kUnit];
    int c[kUnit];
    load8bits(w, base, n, vec, h);
    load8i(ecc, base, n, vec, c);
    float r[kUnit];
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      const int ls = ecc_log_scale_bits<T>(h[i]);
      const int hh = ls >> 1;  // floor(ls / 2)
      const float corr = div_by_code_range((float)c[i], smax);
      const float e = __fmul_rn(__fmul_rn(corr, pow2i(hh)), pow2i(ls - hh));
      r[i] = __fadd_rn(narrow_bits_to_float<T>(h[i]), e);
    }
    store8f(out, base, n, vec, r);
  }
}

template <typename T, typename E>
__global__ void __launch_bounds__(kQThreads) ecc_encode_kernel(const float* __restrict__ x, const T* __restrict__ w,
                                                               E* __restrict__ ecc, int64_t n) {
  const float smax = sizeof(E) == 1 ? 127.0f : 32767.0f;
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  const bool vec = aligned_for_units(x) && aligned_for_units(w) && aligned_for_units(ecc);
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    const int64_t base = unit * kUnit;
    uint16_t h[kUnit];
    float xv[kUnit];
    load8bits(w, base, n, vec, h);
    load8f(x, base, n, vec, xv);
    int c[kUnit];
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      const int neg = -ecc_log_scale_bits<T>(h[i]);
      const int hh = neg >> 1;
      const float e = __fsub_rn(xv[i], narrow_bits_to_float<T>(h[i]));
      float en = __fmul_rn(__fmul_rn(e, pow2i(hh)), pow2i(neg - hh));
      en = fminf(fmaxf(en, -1.0f), 1.0f);
      const float s = __fmul_rn(en, smax);
      c[i] = (int)copysignf(floorf(__fadd_rn(fabsf(s), 0.5f)), s);
    }
    store8i(ecc, base, n, vec, c);
  }
}

template <typename T>
__global__ void __launch_bounds__(kQThreads) maxabs_kernel(const T* __restrict__ x, int64_t n, float* out) {
  float a = 0.0f;
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  const bool vec = aligned_for_units(x);
  for (int64_t unit = (int64_t)blockIdx.x * kQThreads + threadIdx.x; unit < n_units;
       unit += (int64_t)gridDim.x * kQThreads) {
    float v[kUnit];
    load8f(x, unit * kUnit, n, vec, v);
#pragma unroll
    for (int i = 0; i < kUnit; ++i) a = fmaxf(a, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(kFullMask, a, o));
  // non-negative floats order like their bit patterns; NaN inputs are dropped by fmaxf
  if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(a));
}

// Grid: a persistent loop over 16 CTAs per SM (the SM count is read once per device), never
// more than the work.  One unit per thread over the whole grid, like the reference's
// one-block-per-1024-elements launches, was measured too: slower for three of the four
// master-weight kernels (-DFO_QUANT_BLOCKS_PER_SM=k changes the factor for tuning builds).
#ifndef FO_QUANT_BLOCKS_PER_SM
#define FO_QUANT_BLOCKS_PER_SM 16
#endif
static int blocks_for(int64_t units) {
  static int sms[64];
  int dev = 0;
  cudaGetDevice(&dev);
  int n = 148;
  if (dev >= 0 && dev < 64) {
    if (sms[dev] == 0) {
      int v = 0;
      if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
      sms[dev] = v;
    }
    n = sms[dev];
  }
  int64_t b = (units + kQThreads - 1) / kQThreads;
  const int64_t cap = (int64_t)n * FO_QUANT_BLOCKS_PER_SM;
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
  const int grid = fo::blocks_for((n + fo::kUnit - 1) / fo::kUnit);
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
  const int grid = fo::blocks_for((n + fo::kUnit - 1) / fo::kUnit);
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
