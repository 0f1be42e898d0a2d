// Per-unit (8 element) load / update / store of the fused optimizer steps.
//
// What a unit goes through equals one program of the reference's _triton_momentum_kernel
// (flashoptim/optimizers.py:1587-1719: SGD / SGDW / Lion) and _triton_adam_kernel
// (:2256-2443): rebuild the master value from narrow value + correction code, dequantise the
// states, update in fp32, requantise, re-split.
//
// The same three phases serve the plain multi-tensor step kernels and the
// kernels that take their gradient from NVLink peers: those replace only the
// gradient load.
#pragma once

#include "fo_api.h"
#include "fo_common.cuh"

namespace fo {

// Raw register image of one unit of every stream a step touches.
template <typename T, int kErr, int kStates, bool kQ>
struct UnitRegs {
  Raw8<T> p;
  Raw8<T> g;
  uint4 ecc;       // kErr == 1: x,y hold 8 int8; kErr == 2: 8 int16
  uint2 q[2];      // quantised states (codes)
  float sc[2];     // their group scales
  Raw8<T> f[2];    // full-precision states (param dtype)
  int cnt;         // valid elements in this unit: 8, 1..7 (tail) or <= 0 (none)
};

template <typename T>
__device__ __forceinline__ void load_raw8(Raw8<T>& r, const T* base, bool vec) {
  if constexpr (sizeof(T) == 2) {
    if (vec) r.v = ld16_stream(base);
  } else {
    if (vec) {
      r.v = ld16_stream(base);
      r.w = ld16_stream(reinterpret_cast<const char*>(base) + 16);
    }
  }
}
template <typename T>
__device__ __forceinline__ void load_raw8_partial(Raw8<T>& r, const T* base, int cnt) {
  if constexpr (sizeof(T) == 2) {
    uint32_t w[4];
    ld_partial<2, 4>(base, cnt, w);
    r.v = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    uint32_t w[8];
    ld_partial<4, 8>(base, cnt, w);
    r.v = make_uint4(w[0], w[1], w[2], w[3]);
    r.w = make_uint4(w[4], w[5], w[6], w[7]);
  }
}
template <typename T>
__device__ __forceinline__ void store_raw8(const Raw8<T>& r, T* base, int cnt, bool vec) {
  if (vec) {
    st16(base, r.v);
    if constexpr (sizeof(T) == 4) st16(reinterpret_cast<char*>(base) + 16, r.w);
  } else if (cnt > 0) {
    if constexpr (sizeof(T) == 2) {
      const uint32_t w[4] = {r.v.x, r.v.y, r.v.z, r.v.w};
      st_partial<2, 4>(base, cnt, w);
    } else {
      const uint32_t w[8] = {r.v.x, r.v.y, r.v.z, r.v.w, r.w.x, r.w.y, r.w.z, r.w.w};
      st_partial<4, 8>(base, cnt, w);
    }
  }
}

// A segment is "vector safe" when every base pointer is 16-byte aligned; unit
// offsets are multiples of 8 elements, so alignment then holds for every unit.
__device__ __forceinline__ bool seg_vector_safe(const FoSeg& s) {
  uintptr_t a = reinterpret_cast<uintptr_t>(s.p) | reinterpret_cast<uintptr_t>(s.g) |
                reinterpret_cast<uintptr_t>(s.ecc) | reinterpret_cast<uintptr_t>(s.s0) |
                reinterpret_cast<uintptr_t>(s.s1);
  return (a & 15) == 0;
}

// Loads everything except the gradient.
template <typename T, int kErr, int kStates, bool kQ>
__device__ __forceinline__ void load_unit_state(UnitRegs<T, kErr, kStates, kQ>& r, const FoSeg& s,
                                                int64_t base, bool seg_vec) {
  const int64_t left = s.n - base;
  r.cnt = left >= kUnit ? kUnit : (int)left;
  const bool vec = seg_vec && r.cnt == kUnit;
  const bool part = !vec && r.cnt > 0;
  r.p.v = make_uint4(0, 0, 0, 0);
  if constexpr (sizeof(T) == 4) r.p.w = make_uint4(0, 0, 0, 0);
  r.ecc = make_uint4(0, 0, 0, 0);
  const T* pp = static_cast<const T*>(s.p) + base;
  if (vec) load_raw8<T>(r.p, pp, true);
  if (part) load_raw8_partial<T>(r.p, pp, r.cnt);
  if constexpr (kErr == 1) {
    const char* e = static_cast<const char*>(s.ecc) + base;
    if (vec) {
      uint2 t = ld8_stream(e);
      r.ecc.x = t.x;
      r.ecc.y = t.y;
    }
    if (part) {
      uint32_t w[2];
      ld_partial<1, 2>(e, r.cnt, w);
      r.ecc.x = w[0];
      r.ecc.y = w[1];
    }
  } else if constexpr (kErr == 2) {
    const char* e = static_cast<const char*>(s.ecc) + base * 2;
    if (vec) r.ecc = ld16_stream(e);
    if (part) {
      uint32_t w[4];
      ld_partial<2, 4>(e, r.cnt, w);
      r.ecc = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
#pragma unroll
  for (int k = 0; k < kStates; ++k) {
    void* sp = k == 0 ? s.s0 : s.s1;
    void* ss = k == 0 ? s.s0s : s.s1s;
    if constexpr (kQ) {
      r.q[k] = make_uint2(k == 0 ? 0u : 0u, 0u);
      r.sc[k] = 1.0f;
      const char* qp = static_cast<const char*>(sp) + base;
      if (vec) r.q[k] = ld8_stream(qp);
      if (part) {
        uint32_t w[2];
        ld_partial<1, 2>(qp, r.cnt, w);
        r.q[k] = make_uint2(w[0], w[1]);
      }
      if (r.cnt > 0) r.sc[k] = __half2float(static_cast<const __half*>(ss)[base >> 5]);
    } else {
      r.f[k].v = make_uint4(0, 0, 0, 0);
      if constexpr (sizeof(T) == 4) r.f[k].w = make_uint4(0, 0, 0, 0);
      const T* fp = static_cast<const T*>(sp) + base;
      if (vec) load_raw8<T>(r.f[k], fp, true);
      if (part) load_raw8_partial<T>(r.f[k], fp, r.cnt);
    }
  }
}

template <typename T, int kErr, int kStates, bool kQ>
__device__ __forceinline__ void load_unit_grad(UnitRegs<T, kErr, kStates, kQ>& r, const FoSeg& s,
                                               int64_t base, bool seg_vec) {
  const bool vec = seg_vec && r.cnt == kUnit;
  r.g.v = make_uint4(0, 0, 0, 0);
  if constexpr (sizeof(T) == 4) r.g.w = make_uint4(0, 0, 0, 0);
  const T* gp = static_cast<const T*>(s.g) + base;
  if (vec) load_raw8<T>(r.g, gp, true);
  if (!vec && r.cnt > 0) load_raw8_partial<T>(r.g, gp, r.cnt);
}

// Widen parameter (+ correction) and states to fp32.
template <typename T, int kErr, int kStates, bool kQ>
__device__ __forceinline__ void widen_unit(const UnitRegs<T, kErr, kStates, kQ>& r, float2 (&p)[4],
                                           float2 (&m)[4], float2 (&v)[4]) {
  unpack8<T>(r.p, p);
  if constexpr (kErr != 0) {
    float2 c[4];
    ecc_codes_scaled<T, kErr>(r.ecc, c);
    ecc_apply8<T>(p, c);
  }
  if constexpr (kStates >= 1) {
    if constexpr (kQ) dequant_softsign8(r.q[0], r.sc[0], m);
    else unpack8<T>(r.f[0], m);
  }
  if constexpr (kStates >= 2) {
    if constexpr (kQ) dequant_sqrt8(r.q[1], r.sc[1], v);
    else unpack8<T>(r.f[1], v);
  }
}

// Narrow and store parameter, correction and states.  `pn` returns the narrowed
// parameter unit as stored (for callers that also send it elsewhere).
template <typename T, int kErr, int kStates, bool kQ>
__device__ __forceinline__ void store_unit(const UnitRegs<T, kErr, kStates, kQ>& r, const FoSeg& s,
                                           int64_t base, bool seg_vec, const float2 (&p)[4],
                                           const float2 (&m)[4], const float2 (&v)[4], Raw8<T>& pn) {
  // when kQ, `v` holds the square root of the second state (what its codes store)
  const bool vec = seg_vec && r.cnt == kUnit;
  float2 back[4];
  pack8<T>(p, pn, back);
  store_raw8<T>(pn, static_cast<T*>(s.p) + base, r.cnt, vec);
  if constexpr (kErr == 1) {
    float2 sres[4];
    ecc_residual8<T, 1>(p, back, sres);
    uint2 c = round_to_bytes(sres);
    char* e = static_cast<char*>(s.ecc) + base;
    if (vec) st8(e, c);
    else if (r.cnt > 0) {
      const uint32_t w[2] = {c.x, c.y};
      st_partial<1, 2>(e, r.cnt, w);
    }
  } else if constexpr (kErr == 2) {
    float2 sres[4];
    ecc_residual8<T, 2>(p, back, sres);
    uint4 c = round_to_shorts(sres);
    char* e = static_cast<char*>(s.ecc) + base * 2;
    if (vec) st16(e, c);
    else if (r.cnt > 0) {
      const uint32_t w[4] = {c.x, c.y, c.z, c.w};
      st_partial<2, 4>(e, r.cnt, w);
    }
  }
#pragma unroll
  for (int k = 0; k < kStates; ++k) {
    void* sp = k == 0 ? s.s0 : s.s1;
    void* ss = k == 0 ? s.s0s : s.s1s;
    const float2(&x)[4] = k == 0 ? m : v;
    if constexpr (kQ) {
      uint2 codes;
      // every lane takes part in the group shuffle, valid unit or not
      const float a = k == 0 ? quant_softsign8(x, codes) : quant_sqrt8_pre(x, codes);
      char* qp = static_cast<char*>(sp) + base;
      if (vec) st8(qp, codes);
      else if (r.cnt > 0) {
        const uint32_t w[2] = {codes.x, codes.y};
        st_partial<1, 2>(qp, r.cnt, w);
      }
      // the first lane of a group always holds valid elements if any lane does
      if ((threadIdx.x & 3) == 0 && r.cnt > 0) static_cast<__half*>(ss)[base >> 5] = __float2half_rn(a);
    } else {
      Raw8<T> fn;
      float2 unused[4];
      pack8<T>(x, fn, unused);
      store_raw8<T>(fn, static_cast<T*>(sp) + base, r.cnt, vec);
    }
  }
}

template <typename T, int kErr, int kStates, bool kQ>
__device__ __forceinline__ void store_unit(const UnitRegs<T, kErr, kStates, kQ>& r, const FoSeg& s,
                                           int64_t base, bool seg_vec, const float2 (&p)[4],
                                           const float2 (&m)[4], const float2 (&v)[4]) {
  Raw8<T> pn;
  store_unit(r, s, base, seg_vec, p, m, v, pn);
}

// ---------------------------------------------------------------- update rules on 8 elements

// Adam / AdamW.  On return `v` holds the new second moment, or its square root
// when kSqrtOut (the quantised state stores sqrt(v), and the denominator needs
// the same square root: one evaluation serves both).
template <bool kSqrtOut>
__device__ __forceinline__ void adam_update8(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4],
                                             float2 (&v)[4], const FoAdamHyper& h) {
  const float2 b1 = splat2(h.beta1), b2 = splat2(h.beta2);
  const float2 c1 = splat2(h.one_minus_beta1 * h.grad_scale);
  const float2 step = splat2(-h.lr * h.rbc1);
  const float2 srbc2 = splat2(h.sqrt_rbc2), eps = splat2(h.eps);
  if (h.decoupled) {
    const float2 c2 = splat2(h.one_minus_beta2 * h.grad_scale * h.grad_scale);
    const float2 decay = splat2(h.decay);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      m[i] = fma2(m[i], b1, mul2(g[i], c1));
      float2 vn = fma2(v[i], b2, mul2(mul2(g[i], g[i]), c2));
      float2 sv = make_float2(fast_sqrt(vn.x), fast_sqrt(vn.y));
      float2 den = fma2(sv, srbc2, eps);
      den = make_float2(fast_rcp(den.x), fast_rcp(den.y));
      p[i] = fma2(mul2(m[i], step), den, mul2(p[i], decay));
      v[i] = kSqrtOut ? sv : vn;
    }
  } else {
    const float2 gs = splat2(h.grad_scale), l2 = splat2(h.weight_decay);
    const float2 omb1 = splat2(h.one_minus_beta1), omb2 = splat2(h.one_minus_beta2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 gi = fma2(p[i], l2, mul2(g[i], gs));
      m[i] = fma2(m[i], b1, mul2(gi, omb1));
      float2 vn = fma2(v[i], b2, mul2(mul2(gi, gi), omb2));
      float2 sv = make_float2(fast_sqrt(vn.x), fast_sqrt(vn.y));
      float2 den = fma2(sv, srbc2, eps);
      den = make_float2(fast_rcp(den.x), fast_rcp(den.y));
      p[i] = fma2(mul2(m[i], step), den, p[i]);
      v[i] = kSqrtOut ? sv : vn;
    }
  }
}

__device__ __forceinline__ void momentum_update8(float2 (&p)[4], const float2 (&g)[4], float2 (&m)[4],
                                                 const FoMomentumHyper& h, bool has_state) {
  const float2 mc = splat2(h.mom_coef);
  if (h.lion) {
    const float2 uc = splat2(h.update_coef);
    const float2 omuc = splat2(h.one_minus_update_coef * h.grad_scale);
    const float2 ommc = splat2(h.one_minus_mom_coef * h.grad_scale);
    const float2 decay = splat2(h.decay);
    const uint32_t lr_bits = __float_as_uint(h.lr);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 c = fma2(m[i], uc, mul2(g[i], omuc));
      m[i] = fma2(m[i], mc, mul2(g[i], ommc));
      // -lr * sign(c): lr with the flipped sign bit of c, or 0 when c == 0
      float2 u;
      u.x = c.x == 0.0f ? 0.0f : __uint_as_float(lr_bits | (~__float_as_uint(c.x) & 0x80000000u));
      u.y = c.y == 0.0f ? 0.0f : __uint_as_float(lr_bits | (~__float_as_uint(c.y) & 0x80000000u));
      p[i] = fma2(p[i], decay, u);
    }
    return;
  }
  const float2 decay = splat2(h.decay);
  const float2 l2 = splat2(h.decoupled ? 0.0f : h.weight_decay);
  const float2 gs = splat2(h.grad_scale);
  const float2 ucoef = splat2(h.update_coef);
  const float2 nlr = splat2(-h.lr);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 gi = fma2(p[i], l2, mul2(g[i], gs));
    float2 pd = mul2(p[i], decay);
    if (!has_state) {
      p[i] = fma2(gi, nlr, pd);
      continue;
    }
    m[i] = fma2(m[i], mc, mul2(gi, ucoef));
    float2 upd = h.nesterov ? fma2(m[i], mc, gi) : m[i];
    p[i] = fma2(upd, nlr, pd);
  }
}

}  // namespace fo
