// Helpers shared by the hybrid-decoder kernels (Dynamic-Tanh norms, state-space scan, sliding-window attention with a
// softmax sink, mixture of experts).  These kernels keep the residual stream, every norm, softmax, router and recurrence
// in fp32; the element type T (bf16 or float) is the type of GEMM operands, KV pools and weights: bf16 when the model is
// served in bf16, float when it runs entirely in 32-bit.
#pragma once
#include "common.cuh"

namespace b200 {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int64_t i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, int64_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

template <typename T>
__device__ __forceinline__ void stf(T* p, int64_t i, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, int64_t i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// exact-exponential SiLU (the fp32 serving mode compares at 1e-5; common.cuh's silu_f32 is the fast-path variant)
// 16-byte asynchronous global -> shared copy; `ok` false writes zeros (source size 0) and reads nothing
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool ok) {
  const int n = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// packed fp32 pairs (sm_100 fma.rn.f32x2 / mul.rn.f32x2): two IEEE fp32 operations per issue slot, each lane rounded exactly
// like the scalar instruction
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rc, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmov.b64 rc, {%6, %7};\n"
      "fma.rn.f32x2 rd, ra, rb, rc;\nmov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2, %3};\nmov.b64 rb, {%4, %5};\nmul.rn.f32x2 rd, ra, rb;\nmov.b64 {%0, %1}, rd;\n}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}


// element-type dispatch: `dt` is B200_BF16 or B200_F32
#define B200_DISPATCH_ELEM(dt, T, ...)                                        \
  do {                                                                        \
    if ((dt) == B200_BF16) {                                                  \
      using T = __nv_bfloat16;                                                \
      __VA_ARGS__;                                                            \
    } else if ((dt) == B200_F32) {                                            \
      using T = float;                                                        \
      __VA_ARGS__;                                                            \
    } else {                                                                  \
      ::b200::set_last_error("element type %d is neither bf16 nor f32", dt);  \
      return B200_ERR_INVALID_ARG;                                            \
    }                                                                         \
  } while (0)

}  // namespace b200
