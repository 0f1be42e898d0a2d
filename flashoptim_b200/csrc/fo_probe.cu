// Test-support entry points: the FAST forms of the master-weight split (the device functions
// that the step kernels inline, fo_common.cuh) applied to arbitrary fp32 inputs.
//
// Inside a step kernel the value that gets split is the result of an update, so a test cannot
// feed it every fp32 bit pattern.  These two kernels run exactly the same device functions
// (pack8 + ecc_residual8 + round_to_bytes / round_to_shorts for the split, unpack8 +
// ecc_codes_scaled + ecc_apply8 for the merge) on caller-supplied values, which is what an
// exhaustive sweep over all mantissas needs.  The reference has a test-only kernel for the same
// purpose (test/test_ecc_invariants.py:24-156).  Lengths must be multiples of 8 and pointers
// 16-byte aligned (whole units only); nothing else in the library calls these.
#include "fo_api.h"
#include "fo_step_core.cuh"

namespace fo {

template <typename T, int kErr>
__global__ void __launch_bounds__(256) fast_ecc_split_kernel(const float* __restrict__ x, T* __restrict__ narrow,
                                                             void* __restrict__ ecc, int64_t n_units) {
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < n_units;
       u += (int64_t)gridDim.x * blockDim.x) {
    const int64_t base = u * kUnit;
    Raw8<float> xr;
    xr.v = ld16(x + base);
    xr.w = ld16(x + base + 4);
    float2 xf[4], back[4], s[4];
    unpack8<float>(xr, xf);
    Raw8<T> pn;
    pack8<T>(xf, pn, back);
    st16(narrow + base, pn.v);
    ecc_residual8<T, kErr>(xf, back, s);
    if constexpr (kErr == 1) st8(static_cast<char*>(ecc) + base, round_to_bytes(s));
    else st16(static_cast<char*>(ecc) + base * 2, round_to_shorts(s));
  }
}

template <typename T, int kErr>
__global__ void __launch_bounds__(256) fast_ecc_merge_kernel(const T* __restrict__ narrow, const void* __restrict__ ecc,
                                                             float* __restrict__ out, int64_t n_units) {
  for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < n_units;
       u += (int64_t)gridDim.x * blockDim.x) {
    const int64_t base = u * kUnit;
    Raw8<T> pr;
    pr.v = ld16(narrow + base);
    uint4 codes = make_uint4(0, 0, 0, 0);
    if constexpr (kErr == 1) {
      const uint2 c = ld8(static_cast<const char*>(ecc) + base);
      codes.x = c.x;
      codes.y = c.y;
    } else {
      codes = ld16(static_cast<const char*>(ecc) + base * 2);
    }
    float2 p[4], c[4], unused[4];
    unpack8<T>(pr, p);
    ecc_codes_scaled<T, kErr>(codes, c);
    ecc_apply8<T>(p, c);
    Raw8<float> o;
    pack8<float>(p, o, unused);
    st16(out + base, o.v);
    st16(out + base + 4, o.w);
  }
}

static bool probe_args_ok(const void* a, const void* b, const void* c, int64_t n) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
  return a && b && c && n >= 0 && (n % kUnit) == 0 && (bits & 15) == 0;
}

}  // namespace fo

extern "C" int fo_probe_fast_ecc_split(const float* x, int dtype, int err_bytes, void* narrow, void* ecc,
                                       int64_t n, void* stream) {
  if (!fo::probe_args_ok(x, narrow, ecc, n)) return (int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  const int64_t units = n / fo::kUnit;
  const int grid = (int)((units + 255) / 256 < 148 * 16 ? (units + 255) / 256 : 148 * 16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FO_BF16 && err_bytes == 1)
    fo::fast_ecc_split_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>(x, (__nv_bfloat16*)narrow, ecc, units);
  else if (dtype == FO_BF16 && err_bytes == 2)
    fo::fast_ecc_split_kernel<__nv_bfloat16, 2><<<grid, 256, 0, st>>>(x, (__nv_bfloat16*)narrow, ecc, units);
  else if (dtype == FO_FP16 && err_bytes == 1)
    fo::fast_ecc_split_kernel<__half, 1><<<grid, 256, 0, st>>>(x, (__half*)narrow, ecc, units);
  else if (dtype == FO_FP16 && err_bytes == 2)
    fo::fast_ecc_split_kernel<__half, 2><<<grid, 256, 0, st>>>(x, (__half*)narrow, ecc, units);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

extern "C" int fo_probe_fast_ecc_merge(const void* narrow, int dtype, const void* ecc, int err_bytes, float* out,
                                       int64_t n, void* stream) {
  if (!fo::probe_args_ok(narrow, ecc, out, n)) return (int)cudaErrorInvalidValue;
  if (n == 0) return 0;
  const int64_t units = n / fo::kUnit;
  const int grid = (int)((units + 255) / 256 < 148 * 16 ? (units + 255) / 256 : 148 * 16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == FO_BF16 && err_bytes == 1)
    fo::fast_ecc_merge_kernel<__nv_bfloat16, 1><<<grid, 256, 0, st>>>((const __nv_bfloat16*)narrow, ecc, out, units);
  else if (dtype == FO_BF16 && err_bytes == 2)
    fo::fast_ecc_merge_kernel<__nv_bfloat16, 2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)narrow, ecc, out, units);
  else if (dtype == FO_FP16 && err_bytes == 1)
    fo::fast_ecc_merge_kernel<__half, 1><<<grid, 256, 0, st>>>((const __half*)narrow, ecc, out, units);
  else if (dtype == FO_FP16 && err_bytes == 2)
    fo::fast_ecc_merge_kernel<__half, 2><<<grid, 256, 0, st>>>((const __half*)narrow, ecc, out, units);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}
