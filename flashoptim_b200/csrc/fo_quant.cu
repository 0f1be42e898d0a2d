// Stand-alone group quantiser / dequantiser, master-weight split and maxabs.
//
// These run at checkpoint save/load, fp32 export/import and when a state is set
// from a full-precision tensor (never inside a training step), so
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
// Register budgets (launch bounds) that measured best on B200: 32 registers (8 CTAs per SM) for
// the quantiser and dequantiser, 40 (6 CTAs, nothing spilled) for the master-weight kernels.
constexpr int kQuantMinBlocks = 8;
constexpr int kEccMinBlocks = 6;

// ---------------------------------------------------------------- memory access
// Read-once data through the non-coherent path with default caching: measured 2-3 % faster in
// these kernels than L1::no_allocate loads.
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg8(const void* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ uint32_t ldg4(const void* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }

// 256-bit accesses (sm_100 and later): a unit of eight fp32 values is one request.
struct Words8 {
  uint32_t w[8];
};
__device__ __forceinline__ bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }
__device__ __forceinline__ Words8 ldg32(const void* p) {
  Words8 v;
  asm volatile("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]),
                 "=r"(v.w[7])
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st32(void* p, const Words8& v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]),
               "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
               : "memory");
}

// The quantiser and dequantiser give a thread one unit of 8 consecutive elements per iteration
// (four lanes form a group of 32) and move it with vector accesses when the tensor's base
// address allows and the unit is whole: 32 bytes for fp32 (two 16-byte requests when the unit
// is only 16-byte aligned), 16 for 2-byte and 8 for 1-byte elements.  Tails and unaligned
// tensors go element by element.  The arithmetic per element is the same in both paths.

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
      if (aligned32(p + base)) {
        const Words8 a = ldg32(p + base);
#pragma unroll
        for (int i = 0; i < kUnit; ++i) v[i] = __uint_as_float(a.w[i]);
      } else {
        const uint4 a = ldg16(p + base), b = ldg16(p + base + 4);
        v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
        v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
      }
    } else {
      const uint4 a = ldg16(p + base);
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
__device__ __forceinline__ void store8f(float* p, int64_t base, int64_t n, bool vec, const float (&v)[kUnit]) {
  if (vec && base + kUnit <= n) {
    if (aligned32(p + base)) {
      Words8 o;
#pragma unroll
      for (int i = 0; i < kUnit; ++i) o.w[i] = __float_as_uint(v[i]);
      st32(p + base, o);
    } else {
      st16(p + base, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
      st16(p + base + 4,
           make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
    }
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i)
      if (base + i < n) p[base + i] = v[i];
  }
}
// 8 one-byte integers (two's complement in the low bits of c[i]).
template <typename E>
__device__ __forceinline__ void store8i(E* p, int64_t base, int64_t n, bool vec, const int (&c)[kUnit]) {
  static_assert(sizeof(E) == 1, "8-bit codes only");
  if (vec && base + kUnit <= n) {
    uint2 o;
    o.x = (c[0] & 0xff) | ((c[1] & 0xff) << 8) | ((c[2] & 0xff) << 16) | ((uint32_t)(c[3] & 0xff) << 24);
    o.y = (c[4] & 0xff) | ((c[5] & 0xff) << 8) | ((c[6] & 0xff) << 16) | ((uint32_t)(c[7] & 0xff) << 24);
    st8(p + base, o);
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i)
      if (base + i < n) p[base + i] = (E)c[i];
  }
}
template <typename E>
__device__ __forceinline__ void load8i(const E* p, int64_t base, int64_t n, bool vec, int (&c)[kUnit]) {
  static_assert(sizeof(E) == 1, "8-bit codes only");
  if (vec && base + kUnit <= n) {
    const uint2 a = ldg8(p + base);
    const uint32_t w[2] = {a.x, a.y};
#pragma unroll
    for (int i = 0; i < kUnit; ++i) {
      const uint32_t b = (w[i >> 2] >> (8 * (i & 3))) & 0xffu;
      c[i] = std::is_signed<E>::value ? (int)(int8_t)b : (int)b;
    }
  } else {
#pragma unroll
    for (int i = 0; i < kUnit; ++i) c[i] = base + i < n ? (int)p[base + i] : 0;
  }
}

// One thread per unit of 8 elements; four lanes form a group.
template <typename T, bool kSigned, bool kSqrt, bool kSoftsign>
__global__ void __launch_bounds__(kQThreads, kQuantMinBlocks)
    quantize_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, __half* __restrict__ scales, int64_t n) {
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
__global__ void __launch_bounds__(kQThreads, kQuantMinBlocks)
    dequantize_kernel(const uint8_t* __restrict__ q, const __half* __restrict__ scales, float* __restrict__ out,
                      int64_t n) {
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

// ---------------------------------------------------------------- master-weight split / merge

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

// 2^ls and 2^-ls (ls = E(w) - M - 1) as single floats, straight from the exponent field of the
// narrow value.  The PyTorch formulation scales by two powers of two so that nothing under- or
// overflows on the way; one factor gives the same bits whenever it is itself a normal number and
// the scaled correction is (an exact scaling then, and `code * 2^ls + w` rounds once either
// way).  fp16: always (E >= -14; subnormals and zero share the smallest normal's exponent, the
// clamp).  bf16: for |w| >= 2^-94; smaller values, zero included, take the two-factor form.
template <typename T>
__device__ __forceinline__ bool single_scale_ok(float w) {
  if constexpr (std::is_same<T, __half>::value) return true;
  else return fabsf(w) >= 5.048709793414476e-29f;  // 2^-94; false for NaN
}
template <typename T>
__device__ __forceinline__ float ecc_scale(uint16_t bits) {
  if constexpr (std::is_same<T, __half>::value)
    return __uint_as_float((max((uint32_t)bits & 0x7C00u, 0x0400u) << 13) + ((127u - 15u - 11u) << 23));
  else
    return __uint_as_float((((uint32_t)bits << 16) & 0x7F800000u) - (8u << 23));
}
template <typename T>
__device__ __forceinline__ float ecc_inv_scale(uint16_t bits) {
  if constexpr (std::is_same<T, __half>::value)
    return __uint_as_float(((127u + 15u + 11u) << 23) - (max((uint32_t)bits & 0x7C00u, 0x0400u) << 13));
  else
    return __uint_as_float(((254u + 8u) << 23) - (((uint32_t)bits << 16) & 0x7F800000u));
}

// The split / merge kernels use an interleaved layout: a warp owns a tile of 256 consecutive
// elements and a lane moves elements [4 * lane, 4 * lane + 4) of each half, so that every
// warp-wide access covers one contiguous span (512 / 256 / 128 bytes for 4- / 2- / 1-byte
// elements).  Measured against 8 consecutive elements per lane (32-byte fp32 accesses at a
// 32-byte stride): 4-15 % faster.
template <typename T>
__device__ __forceinline__ bool aligned_for_quads(const T* p) {
  return (reinterpret_cast<uintptr_t>(p) & (sizeof(T) * 4 - 1)) == 0;
}
// Four elements as sizeof(T) packed words; zero beyond n.
template <typename T>
__device__ __forceinline__ void load4raw(const T* p, int64_t base, int64_t n, bool vec, uint32_t (&w)[sizeof(T)]) {
  if (vec && base + 4 <= n) {
    if constexpr (sizeof(T) == 4) {
      const uint4 a = ldg16(p + base);
      w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    } else if constexpr (sizeof(T) == 2) {
      const uint2 a = ldg8(p + base);
      w[0] = a.x; w[1] = a.y;
    } else {
      w[0] = ldg4(p + base);
    }
  } else {
#pragma unroll
    for (int k = 0; k < (int)sizeof(T); ++k) w[k] = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (base + i < n) {
        if constexpr (sizeof(T) == 4) w[i] = reinterpret_cast<const uint32_t*>(p)[base + i];
        else if constexpr (sizeof(T) == 2)
          w[i >> 1] |= (uint32_t) reinterpret_cast<const uint16_t*>(p)[base + i] << (16 * (i & 1));
        else w[0] |= (uint32_t) reinterpret_cast<const uint8_t*>(p)[base + i] << (8 * i);
      }
    }
  }
}
template <typename T>
__device__ __forceinline__ void store4raw(T* p, int64_t base, int64_t n, bool vec, const uint32_t (&w)[sizeof(T)]) {
  if (vec && base + 4 <= n) {
    if constexpr (sizeof(T) == 4) st16(p + base, make_uint4(w[0], w[1], w[2], w[3]));
    else if constexpr (sizeof(T) == 2) st8(p + base, make_uint2(w[0], w[1]));
    else *reinterpret_cast<uint32_t*>(p + base) = w[0];
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (base + i < n) {
        if constexpr (sizeof(T) == 4) reinterpret_cast<uint32_t*>(p)[base + i] = w[i];
        else if constexpr (sizeof(T) == 2)
          reinterpret_cast<uint16_t*>(p)[base + i] = (uint16_t)(w[i >> 1] >> (16 * (i & 1)));
        else reinterpret_cast<uint8_t*>(p)[base + i] = (uint8_t)(w[0] >> (8 * i));
      }
    }
  }
}
// Element i of a packed quad of signed codes as an exact float.  The caller has flipped the sign
// bit of every code in the packed word (code + 128, or + 32768, as an unsigned field); one byte
// permute drops that field into the mantissa of 2^23 and subtracting 2^23 + the offset leaves
// the code: no integer-to-float conversion and no sign extension per element.
template <typename E>
__device__ __forceinline__ float quad_code_f(const uint32_t (&w)[sizeof(E)], int i) {
  if constexpr (sizeof(E) == 1)
    return __fsub_rn(__uint_as_float(__byte_perm(w[0], 0x4B000000u, 0x7440u | i)), 8388736.0f);
  else
    return __fsub_rn(__uint_as_float(__byte_perm(w[i >> 1], 0x4B000000u, (i & 1) ? 0x7432u : 0x7410u)), 8421376.0f);
}

template <typename T, typename E>
__global__ void __launch_bounds__(kQThreads, kEccMinBlocks)
    ecc_decode_kernel(const T* __restrict__ w, const E* __restrict__ ecc, float* __restrict__ out, int64_t n) {
  const float smax = sizeof(E) == 1 ? 127.0f : 32767.0f;
  const uint32_t flip = sizeof(E) == 1 ? 0x80808080u : 0x80008000u;
  const bool vec = aligned_for_quads(w) && aligned_for_quads(ecc) && aligned_for_quads(out);
  const int lane = threadIdx.x & 31;
  const int64_t n_tiles = (n + 255) >> 8;
  const int64_t n_warps = (int64_t)gridDim.x * (kQThreads / 32);
  for (int64_t tile = ((int64_t)blockIdx.x * kQThreads + threadIdx.x) >> 5; tile < n_tiles; tile += n_warps) {
    const int64_t b[2] = {tile * 256 + lane * 4, tile * 256 + 128 + lane * 4};
    uint32_t wn[2][2], wc[2][sizeof(E)];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      load4raw(w, b[hf], n, vec, wn[hf]);
      load4raw(ecc, b[hf], n, vec, wc[hf]);
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
      for (int k = 0; k < (int)sizeof(E); ++k) wc[hf][k] ^= flip;
      uint32_t r[4];
      uint16_t hb[4];
      float wf[4];
      bool single = true;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hb[i] = (uint16_t)(wn[hf][i >> 1] >> (16 * (i & 1)));
        wf[i] = narrow_bits_to_float<T>(hb[i]);
        single = single && single_scale_ok<T>(wf[i]);
      }
      if (single) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float corr = div_by_code_range(quad_code_f<E>(wc[hf], i), smax);
          r[i] = __float_as_uint(__fmaf_rn(corr, ecc_scale<T>(hb[i]), wf[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ls = ecc_log_scale_bits<T>(hb[i]);
          const int hh = ls >> 1;  // floor(ls / 2)
          const float corr = div_by_code_range(quad_code_f<E>(wc[hf], i), smax);
          const float e = __fmul_rn(__fmul_rn(corr, pow2i(hh)), pow2i(ls - hh));
          r[i] = __float_as_uint(__fadd_rn(wf[i], e));
        }
      }
      store4raw(out, b[hf], n, vec, r);
    }
  }
}

template <typename T, typename E>
__global__ void __launch_bounds__(kQThreads, kEccMinBlocks)
    ecc_encode_kernel(const float* __restrict__ x, const T* __restrict__ w, E* __restrict__ ecc, int64_t n) {
  const float smax = sizeof(E) == 1 ? 127.0f : 32767.0f;
  const bool vec = aligned_for_quads(x) && aligned_for_quads(w) && aligned_for_quads(ecc);
  const int lane = threadIdx.x & 31;
  const int64_t n_tiles = (n + 255) >> 8;
  const int64_t n_warps = (int64_t)gridDim.x * (kQThreads / 32);
  for (int64_t tile = ((int64_t)blockIdx.x * kQThreads + threadIdx.x) >> 5; tile < n_tiles; tile += n_warps) {
    const int64_t b[2] = {tile * 256 + lane * 4, tile * 256 + 128 + lane * 4};
    uint32_t wn[2][2], wx[2][4];
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      load4raw(w, b[hf], n, vec, wn[hf]);
      load4raw(x, b[hf], n, vec, wx[hf]);
    }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t o[sizeof(E)];
#pragma unroll
      for (int k = 0; k < (int)sizeof(E); ++k) o[k] = 0;
      uint16_t hb[4];
      float wf[4];
      bool single = true;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        hb[i] = (uint16_t)(wn[hf][i >> 1] >> (16 * (i & 1)));
        wf[i] = narrow_bits_to_float<T>(hb[i]);
        single = single && single_scale_ok<T>(wf[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float e = __fsub_rn(__uint_as_float(wx[hf][i]), wf[i]);
        float en;
        if (single) {
          en = __fmul_rn(e, ecc_inv_scale<T>(hb[i]));
        } else {
          const int neg = -ecc_log_scale_bits<T>(hb[i]);
          const int hh = neg >> 1;
          en = __fmul_rn(__fmul_rn(e, pow2i(hh)), pow2i(neg - hh));
        }
        en = fminf(fmaxf(en, -1.0f), 1.0f);  // a NaN difference becomes -1
        const float s = __fmul_rn(en, smax);
        // copysign(floor(|s| + 0.5), s) without a float-to-int conversion: for 0 <= t < 2^23,
        // t + 2^23 rounded down leaves floor(t) in the mantissa
        const float t = __fadd_rn(fabsf(s), 0.5f);
        const int mag = __float_as_int(__fadd_rd(t, 8388608.0f)) & 0x7FFFFF;
        const int c = s < 0.0f ? -mag : mag;
        if constexpr (sizeof(E) == 1) o[0] |= (uint32_t)(c & 0xff) << (8 * i);
        else o[i >> 1] |= (uint32_t)(c & 0xffff) << (16 * (i & 1));
      }
      store4raw(ecc, b[hf], n, vec, o);
    }
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

// Grid: a grid-stride loop over at most 128 CTAs per SM (the SM count is read once per device),
// never more than the work.  Measured on B200 with 2^28 elements: a grid of exactly the
// resident CTAs (one round, equal shares) was 10 % slower for the quantiser, because the SMs do
// not all run at the same pace and a fixed share per CTA waits for the slowest; 16 per SM lost
// to round quantisation (2.7-3.2 rounds at a residency of 5-6); 24 / 32 / 48 / 128 per SM got
// faster in that order; one unit per thread over the whole grid (no loop) was slower again for
// five of the seven kernels.  -DFO_QUANT_BLOCKS_PER_SM=k changes the factor for tuning builds.
#ifndef FO_QUANT_BLOCKS_PER_SM
#define FO_QUANT_BLOCKS_PER_SM 128
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
template <auto kKernel, typename... Args>
static void launch_strided(int64_t units, cudaStream_t st, Args... args) {
  kKernel<<<blocks_for(units), kQThreads, 0, st>>>(args...);
}

template <typename T, bool kSigned, bool kSqrt>
static void launch_quant(const void* x, void* q, void* scales, int64_t n, int softsign, cudaStream_t st) {
  const int64_t n_units = ((n + kGroup - 1) / kGroup) * (kGroup / kUnit);
  if (softsign)
    launch_strided<quantize_kernel<T, kSigned, kSqrt, true>>(n_units, st, (const T*)x, (uint8_t*)q, (__half*)scales, n);
  else
    launch_strided<quantize_kernel<T, kSigned, kSqrt, false>>(n_units, st, (const T*)x, (uint8_t*)q, (__half*)scales, n);
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
  const int64_t n_units = (n + kUnit - 1) / kUnit;
  if (softsign)
    launch_strided<dequantize_kernel<kSigned, kSqrt, true>>(n_units, st, (const uint8_t*)q, (const __half*)scales, out, n);
  else
    launch_strided<dequantize_kernel<kSigned, kSqrt, false>>(n_units, st, (const uint8_t*)q, (const __half*)scales, out, n);
}

// The split / merge kernels take 8 elements per thread and iteration as well (two quads).
template <typename T, typename E>
static void launch_decode(const void* narrow, const void* ecc, float* out, int64_t n, cudaStream_t st) {
  launch_strided<ecc_decode_kernel<T, E>>((n + kUnit - 1) / kUnit, st, (const T*)narrow, (const E*)ecc, out, n);
}
template <typename T, typename E>
static void launch_encode(const float* x, const void* narrow, void* ecc, int64_t n, cudaStream_t st) {
  launch_strided<ecc_encode_kernel<T, E>>((n + kUnit - 1) / kUnit, st, x, (const T*)narrow, (E*)ecc, n);
}
template <typename T>
static void launch_maxabs(const void* x, int64_t n, float* out, cudaStream_t st) {
  launch_strided<maxabs_kernel<T>>((n + kUnit - 1) / kUnit, st, (const T*)x, n, out);
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
  if (dtype == FO_BF16 && err_bytes == 1) fo::launch_decode<__nv_bfloat16, int8_t>(narrow, ecc, out, n, st);
  else if (dtype == FO_BF16 && err_bytes == 2) fo::launch_decode<__nv_bfloat16, int16_t>(narrow, ecc, out, n, st);
  else if (dtype == FO_FP16 && err_bytes == 1) fo::launch_decode<__half, int8_t>(narrow, ecc, out, n, st);
  else if (dtype == FO_FP16 && err_bytes == 2) fo::launch_decode<__half, int16_t>(narrow, ecc, out, n, st);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int fo_ecc_encode(const float* x, const void* narrow, int dtype, void* ecc, int err_bytes,
                             int64_t n, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FO_BF16 && err_bytes == 1) fo::launch_encode<__nv_bfloat16, int8_t>(x, narrow, ecc, n, st);
  else if (dtype == FO_BF16 && err_bytes == 2) fo::launch_encode<__nv_bfloat16, int16_t>(x, narrow, ecc, n, st);
  else if (dtype == FO_FP16 && err_bytes == 1) fo::launch_encode<__half, int8_t>(x, narrow, ecc, n, st);
  else if (dtype == FO_FP16 && err_bytes == 2) fo::launch_encode<__half, int16_t>(x, narrow, ecc, n, st);
  else return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int fo_maxabs(const void* x, int dtype, int64_t n, float* out, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FO_BF16: fo::launch_maxabs<__nv_bfloat16>(x, n, out, st); break;
    case FO_FP16: fo::launch_maxabs<__half>(x, n, out, st); break;
    case FO_FP32: fo::launch_maxabs<float>(x, n, out, st); break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaGetLastError();
}
