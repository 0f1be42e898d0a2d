// Shared device code for the sm_100a optimizer kernels.
//
// Counterparts in the reference (all Triton): group quantise / dequantise inside the step
// kernels, flashoptim/optimizers.py:2543-2676; exponent and correction-code device functions,
// :2683-2776.  The forms here are rearranged for instruction count and documented where they
// deviate in the last bit; the exact forms live in fo_quant.cu.
//
// Layout conventions used by every kernel in this library:
//   * a "unit" is 8 consecutive elements handled by one thread, a quarter of a
//     32-element quantisation group, so a group is four adjacent lanes and its
//     absmax is two xor-shuffles;
//   * narrow tensors (bf16 / fp16) move as one 16-byte vector per unit, 8-bit
//     codes as one 8-byte vector, fp16 scales as one 2-byte load per group.
//
// The B200 moves ~6.5 TB/s, i.e. roughly half a trillion AdamW elements per
// second at 12.25 B/element, which leaves about 60 issue slots per element on
// 148 SMs.  The update is therefore written to be cheap in instructions, not
// only in bytes: packed f32x2 arithmetic (FFMA2/FMUL2/FADD2, new on sm_100),
// integer<->float conversion through the mantissa ("magic number") trick
// instead of the quarter-rate conversion unit, one reciprocal per compander
// evaluation, and error-correction scales built by integer arithmetic on the
// exponent field.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fo {

constexpr int kGroup = 32;  // elements per quantisation group
constexpr int kUnit = 8;    // elements per thread per unit
constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------- packed fp32 helpers

__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

__device__ __forceinline__ float fast_rcp(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fast_sqrt(float x) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// ---------------------------------------------------------------- element traits

template <typename T>
struct Elem;

template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kMant = 7;
  static constexpr bool kNarrow = true;
};
template <>
struct Elem<__half> {
  static constexpr int kMant = 10;
  static constexpr bool kNarrow = true;
};
template <>
struct Elem<float> {
  static constexpr int kMant = 23;
  static constexpr bool kNarrow = false;
};

// 8 consecutive elements of a tensor in registers, raw.
template <typename T>
struct Raw8 {
  uint4 v;
};
template <>
struct Raw8<float> {
  uint4 v, w;
};

template <typename T>
__device__ __forceinline__ void unpack8(const Raw8<T>& r, float2 (&x)[4]);

template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const Raw8<__nv_bfloat16>& r, float2 (&x)[4]) {
  const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[i].x = __uint_as_float(w[i] << 16);
    x[i].y = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const Raw8<__half>& r, float2 (&x)[4]) {
  const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    x[i] = __half22float2(h);
  }
}
template <>
__device__ __forceinline__ void unpack8<float>(const Raw8<float>& r, float2 (&x)[4]) {
  x[0] = make_float2(__uint_as_float(r.v.x), __uint_as_float(r.v.y));
  x[1] = make_float2(__uint_as_float(r.v.z), __uint_as_float(r.v.w));
  x[2] = make_float2(__uint_as_float(r.w.x), __uint_as_float(r.w.y));
  x[3] = make_float2(__uint_as_float(r.w.z), __uint_as_float(r.w.w));
}

// Round 8 fp32 values to T (round to nearest even) and also return the rounded
// values widened back to fp32 (needed by the error-correction encoder).
template <typename T>
__device__ __forceinline__ void pack8(const float2 (&x)[4], Raw8<T>& r, float2 (&back)[4]);

template <>
__device__ __forceinline__ void pack8<__nv_bfloat16>(const float2 (&x)[4], Raw8<__nv_bfloat16>& r,
                                                     float2 (&back)[4]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 b = __float22bfloat162_rn(x[i]);
    w[i] = *reinterpret_cast<uint32_t*>(&b);
    back[i].x = __uint_as_float(w[i] << 16);
    back[i].y = __uint_as_float(w[i] & 0xffff0000u);
  }
  r.v = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ void pack8<__half>(const float2 (&x)[4], Raw8<__half>& r, float2 (&back)[4]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 h = __float22half2_rn(x[i]);
    w[i] = *reinterpret_cast<uint32_t*>(&h);
    back[i] = __half22float2(h);
  }
  r.v = make_uint4(w[0], w[1], w[2], w[3]);
}
template <>
__device__ __forceinline__ void pack8<float>(const float2 (&x)[4], Raw8<float>& r, float2 (&back)[4]) {
  r.v = make_uint4(__float_as_uint(x[0].x), __float_as_uint(x[0].y), __float_as_uint(x[1].x),
                   __float_as_uint(x[1].y));
  r.w = make_uint4(__float_as_uint(x[2].x), __float_as_uint(x[2].y), __float_as_uint(x[3].x),
                   __float_as_uint(x[3].y));
#pragma unroll
  for (int i = 0; i < 4; ++i) back[i] = x[i];
}

// ---------------------------------------------------------------- 8-bit / 16-bit codes <-> fp32

// 0x4B000000 is 2^23; an integer k in [0, 2^22) placed in its low mantissa bits
// reads back as the float 2^23 + k.
constexpr uint32_t kMagicBits = 0x4B000000u;
constexpr float kMagic = 8388608.0f;
// 1.5 * 2^23: adding it to a float s with |s| < 2^22 leaves round-to-nearest-
// even(s) as a two's-complement integer in the low mantissa bits.
constexpr float kRoundMagic = 12582912.0f;

// 8 signed int8 codes (two 32-bit words) -> fp32.
__device__ __forceinline__ void s8_to_float(uint2 c, float2 (&x)[4]) {
  const uint32_t w[2] = {c.x ^ 0x80808080u, c.y ^ 0x80808080u};
  const float2 off = splat2(-(kMagic + 128.0f));
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float2 a, b;
    a.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7650));
    a.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7651));
    b.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7652));
    b.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7653));
    x[2 * i] = add2(a, off);
    x[2 * i + 1] = add2(b, off);
  }
}
// 8 unsigned uint8 codes -> fp32.
__device__ __forceinline__ void u8_to_float(uint2 c, float2 (&x)[4]) {
  const uint32_t w[2] = {c.x, c.y};
  const float2 off = splat2(-kMagic);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float2 a, b;
    a.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7650));
    a.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7651));
    b.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7652));
    b.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7653));
    x[2 * i] = add2(a, off);
    x[2 * i + 1] = add2(b, off);
  }
}
// 8 signed int16 codes (four 32-bit words) -> fp32.
__device__ __forceinline__ void s16_to_float(uint4 c, float2 (&x)[4]) {
  const uint32_t w[4] = {c.x ^ 0x80008000u, c.y ^ 0x80008000u, c.z ^ 0x80008000u, c.w ^ 0x80008000u};
  const float2 off = splat2(-(kMagic + 32768.0f));
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a;
    a.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7610));
    a.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7632));
    x[i] = add2(a, off);
  }
}

// Round 8 fp32 values (|s| < 2^22) to nearest integer and keep the low byte.
__device__ __forceinline__ uint2 round_to_bytes(const float2 (&s)[4]) {
  const float2 mg = splat2(kRoundMagic);
  uint32_t z[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 r = add2(s[i], mg);
    z[2 * i] = __float_as_uint(r.x);
    z[2 * i + 1] = __float_as_uint(r.y);
  }
  uint2 out;
  out.x = __byte_perm(__byte_perm(z[0], z[1], 0x0040), __byte_perm(z[2], z[3], 0x0040), 0x5410);
  out.y = __byte_perm(__byte_perm(z[4], z[5], 0x0040), __byte_perm(z[6], z[7], 0x0040), 0x5410);
  return out;
}
// Same, keeping the low 16 bits.
__device__ __forceinline__ uint4 round_to_shorts(const float2 (&s)[4]) {
  const float2 mg = splat2(kRoundMagic);
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 r = add2(s[i], mg);
    w[i] = __byte_perm(__float_as_uint(r.x), __float_as_uint(r.y), 0x5410);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------- error correction (fast form)
//
// x = w + code / S * 2^ls with ls = E(w) - M - 1 (S = 127 or 32767, M the
// mantissa width of the narrow type, E its unbiased exponent).  2^E is the
// narrow value with its mantissa masked off, one AND on the fp32 image, so
//   decode:  x = w + (code * 2^-(M+1) / S) * 2^E
//   encode:  code = round((x - w) * 2^-E * (S * 2^(M+1)))
// For bf16 values below 2^-126 (zero and subnormals) the mask yields 0: their
// correction, at most 2^-134, is dropped on decode and whatever the encoder
// wrote for them is never used.  fp16 subnormals share the exponent of the
// smallest normal, 2^-14, and are clamped there, which is exact.

template <typename T, int kErrBytes>
struct EccConst {
  static constexpr float kS = kErrBytes == 1 ? 127.0f : 32767.0f;
  static constexpr float kHalfUlp = Elem<T>::kMant == 7 ? 0.00390625f : 0.00048828125f;  // 2^-(M+1)
  static constexpr float kDec = kHalfUlp / kS;
  static constexpr float kEnc = kS / kHalfUlp;
};

// fp32 exponent field of a narrow value that was widened to fp32, i.e. the bits of 2^E.
//   bf16: the value's own field.  Zero and bf16 subnormals have field 0, which reads back as
//         the float 0: on decode their correction (at most 2^-134) is dropped; the encoder
//         still writes some finite code for them, which no decode ever uses.
//   fp16: clamped from below at 113, the field of 2^-14: fp16 subnormals (and zero) share the
//         exponent of the smallest normal, so the clamp is exact.
template <typename T>
__device__ __forceinline__ uint32_t exp_field(float w_as_f32) {
  uint32_t f = __float_as_uint(w_as_f32) & 0x7F800000u;
  if constexpr (Elem<T>::kMant == 10) f = max(f, 113u << 23);
  return f;
}

// 8 signed codes (int8: two words, int16: four words) scaled by kDec, as fp32.
template <typename T, int kErrBytes>
__device__ __forceinline__ void ecc_codes_scaled(uint4 c, float2 (&q)[4]) {
  constexpr float k = EccConst<T, kErrBytes>::kDec;
  if constexpr (kErrBytes == 1) {
    const uint32_t w[2] = {c.x ^ 0x80808080u, c.y ^ 0x80808080u};
    // the offset 2^23 + 128 is subtracted exactly first: folding it into an FMA
    // with k would round (2^23 + 128) * k and shift every code by up to a quarter step
    const float2 kk = splat2(k), off = splat2(-(kMagic + 128.0f));
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float2 a, b;
      a.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7650));
      a.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7651));
      b.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7652));
      b.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7653));
      q[2 * i] = mul2(add2(a, off), kk);
      q[2 * i + 1] = mul2(add2(b, off), kk);
    }
  } else {
    float2 t[4];
    s16_to_float(c, t);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = mul2(t[i], splat2(k));
  }
}

// Master value from narrow value (already widened) + scaled codes.
template <typename T>
__device__ __forceinline__ void ecc_apply8(float2 (&w)[4], const float2 (&code_scaled)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 e2 = make_float2(__uint_as_float(exp_field<T>(w[i].x)), __uint_as_float(exp_field<T>(w[i].y)));
    w[i] = fma2(code_scaled[i], e2, w[i]);
  }
}
// Residual of x against its rounding, in code units (not yet rounded to integer).
template <typename T, int kErrBytes>
__device__ __forceinline__ void ecc_residual8(const float2 (&x)[4], const float2 (&rounded)[4],
                                              float2 (&s)[4]) {
  const float2 neg1 = splat2(-1.0f);
  const float2 kenc = splat2(EccConst<T, kErrBytes>::kEnc);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 e = fma2(rounded[i], neg1, x[i]);  // exact: |e| <= half an ULP of the rounding
    // 2^-E: exponent field 254 - field(w)
    float2 r = make_float2(__uint_as_float(0x7F000000u - exp_field<T>(rounded[i].x)),
                           __uint_as_float(0x7F000000u - exp_field<T>(rounded[i].y)));
    s[i] = mul2(mul2(e, r), kenc);
  }
}

// ---------------------------------------------------------------- group quantisation (fast form)

// absmax over the four lanes of a group.
__device__ __forceinline__ float group_max(float a) {
  a = fmaxf(a, __shfl_xor_sync(kFullMask, a, 1));
  a = fmaxf(a, __shfl_xor_sync(kFullMask, a, 2));
  return a;
}

// Signed companded codes -> fp32: x = scale * q / (254 - |q|).
__device__ __forceinline__ void dequant_softsign8(uint2 codes, float scale, float2 (&x)[4]) {
  float2 q[4];
  s8_to_float(codes, q);
  const float2 sc = splat2(scale);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 r = make_float2(fast_rcp(254.0f - fabsf(q[i].x)), fast_rcp(254.0f - fabsf(q[i].y)));
    x[i] = mul2(mul2(q[i], sc), r);
  }
}
// Unsigned sqrt-domain codes -> fp32: x = (scale * q / 255)^2.
__device__ __forceinline__ void dequant_sqrt8(uint2 codes, float scale, float2 (&x)[4]) {
  const uint32_t w[2] = {codes.x, codes.y};
  const float k = scale * (1.0f / 255.0f);
  const float2 kk = splat2(k), off = splat2(-kMagic * k);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float2 a, b;
    a.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7650));
    a.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7651));
    b.x = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7652));
    b.y = __uint_as_float(__byte_perm(w[i], kMagicBits, 0x7653));
    float2 ra = fma2(a, kk, off), rb = fma2(b, kk, off);
    x[2 * i] = mul2(ra, ra);
    x[2 * i + 1] = mul2(rb, rb);
  }
}

// fp32 -> signed companded codes; returns the group's absmax (the scale).
__device__ __forceinline__ float quant_softsign8(const float2 (&x)[4], uint2& codes) {
  float a = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) a = fmaxf(a, fmaxf(fabsf(x[i].x), fabsf(x[i].y)));
  a = fmaxf(group_max(a), 1e-12f);
  float2 s[4];
  const float inv254 = 1.0f / 254.0f;
  const float a254 = a * inv254;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // 127 * 2n / (1 + |n|) with n = x / a  ==  x / ((a + |x|) / 254)
    float2 r = make_float2(fast_rcp(fmaf(fabsf(x[i].x), inv254, a254)),
                           fast_rcp(fmaf(fabsf(x[i].y), inv254, a254)));
    s[i] = mul2(x[i], r);
  }
  codes = round_to_bytes(s);
  return a;
}
// sqrt-domain values (>= 0, already square-rooted) -> unsigned codes; returns the scale.
__device__ __forceinline__ float quant_sqrt8_pre(const float2 (&r)[4], uint2& codes) {
  float a = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) a = fmaxf(a, fmaxf(r[i].x, r[i].y));
  a = fmaxf(group_max(a), 1e-12f);
  const float2 k = splat2(255.0f * fast_rcp(a));
  float2 s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) s[i] = mul2(r[i], k);
  codes = round_to_bytes(s);
  return a;
}

// ---------------------------------------------------------------- global memory access

__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint2 ld8(const void* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
__device__ __forceinline__ void st8(void* p, uint2 v) { *reinterpret_cast<uint2*>(p) = v; }

// Streaming (read-once) variants: do not keep the line in L1.
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld8_stream(const void* p) {
  uint2 v;
  asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Load / store the first `cnt` (<= 8) elements of a unit one element at a time
// into / from a zero-filled register image.  Slow path for tails and for
// tensors whose base address is not vector aligned; indices are compile-time
// so the image stays in registers.
template <int kBytesPerElem, int kWords>
__device__ __forceinline__ void ld_partial(const void* base, int cnt, uint32_t (&w)[kWords]) {
#pragma unroll
  for (int i = 0; i < kWords; ++i) w[i] = 0;
#pragma unroll
  for (int i = 0; i < kUnit; ++i) {
    if (i < cnt) {
      uint32_t e;
      if constexpr (kBytesPerElem == 1) e = static_cast<const uint8_t*>(base)[i];
      else if constexpr (kBytesPerElem == 2) e = static_cast<const uint16_t*>(base)[i];
      else e = static_cast<const uint32_t*>(base)[i];
      w[(i * kBytesPerElem) >> 2] |= e << (8 * ((i * kBytesPerElem) & 3));
    }
  }
}
template <int kBytesPerElem, int kWords>
__device__ __forceinline__ void st_partial(void* base, int cnt, const uint32_t (&w)[kWords]) {
#pragma unroll
  for (int i = 0; i < kUnit; ++i) {
    if (i < cnt) {
      const uint32_t e = w[(i * kBytesPerElem) >> 2] >> (8 * ((i * kBytesPerElem) & 3));
      if constexpr (kBytesPerElem == 1) static_cast<uint8_t*>(base)[i] = (uint8_t)e;
      else if constexpr (kBytesPerElem == 2) static_cast<uint16_t*>(base)[i] = (uint16_t)e;
      else static_cast<uint32_t*>(base)[i] = e;
    }
  }
}

}  // namespace fo
