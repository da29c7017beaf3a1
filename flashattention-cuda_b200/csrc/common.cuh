// Shared host/device helpers for libfa_b200: status plumbing, small PTX wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/fa_b200.h"

namespace fa {

// ---- error text (thread local) -------------------------------------------------------------------
char* last_error_buf();
int fail(int code, const char* fmt, ...);

#define FA_CHECK_ARG(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::fa::fail(FA_ERR_INVALID, __VA_ARGS__);  \
  } while (0)

#define FA_CUDA_OK(expr)                                                                          \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess)                                                                        \
      return ::fa::fail(FA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),      \
                        __FILE__, __LINE__);                                                      \
  } while (0)

int device_sm_count();  // cached per device; <= 0 on failure

// ---- device helpers ------------------------------------------------------------------------------
#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared, zero-filling when src_bytes == 0.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8,f32) += A(16x16) * B(16x8); A row-major fragments, B column fragments.
template <bool BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// Same product when only rows 0..7 of the 16-row tile are real: the A registers of rows 8..15 and their
// accumulators are zero on input and the results for those rows are dropped.
template <bool BF16, bool R8>
__device__ __forceinline__ void mma_rows(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (!R8) {
    mma16816<BF16>(c, a, b0, b1);
  } else {
    float d2, d3;
    const uint32_t z = 0u;
    const float zf = 0.f;
    if constexpr (BF16) {
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%10,%11,%12,%13};\n"
          : "=f"(c[0]), "=f"(c[1]), "=f"(d2), "=f"(d3)
          : "r"(a[0]), "r"(z), "r"(a[2]), "r"(z), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(zf), "f"(zf));
    } else {
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%10,%11,%12,%13};\n"
          : "=f"(c[0]), "=f"(c[1]), "=f"(d2), "=f"(d3)
          : "r"(a[0]), "r"(z), "r"(a[2]), "r"(z), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(zf), "f"(zf));
    }
  }
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// two E4M3 bytes (low 16 bits of x) -> half2 (low byte -> low half)
__device__ __forceinline__ uint32_t e4m3x2_to_h2(uint32_t x) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.u16.u32 t, %1; cvt.rn.f16x2.e4m3x2 %0, t; }\n" : "=r"(r) : "r"(x));
  return r;
}
// four E4M3 bytes of x -> two half2: lo from bytes 0,1 and hi from bytes 2,3 (the 16-bit halves of the
// register are named directly, no shift)
__device__ __forceinline__ void e4m3x4_to_h2x2(uint32_t x, uint32_t& lo, uint32_t& hi) {
  asm("{ .reg .b16 a, b;\n"
      "  mov.b32 {a, b}, %2;\n"
      "  cvt.rn.f16x2.e4m3x2 %0, a;\n"
      "  cvt.rn.f16x2.e4m3x2 %1, b; }\n"
      : "=r"(lo), "=r"(hi)
      : "r"(x));
}
// four E2M1-pair bytes of x -> four half2 (byte i -> h[i]; low nibble -> low half)
__device__ __forceinline__ void e2m1x8_to_h2x4(uint32_t x, uint32_t (&h)[4]) {
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      "  mov.b32 {b0, b1, b2, b3}, %4;\n"
      "  cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "  cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "  cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "  cvt.rn.f16x2.e2m1x2 %3, b3; }\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(x));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.f16x2 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__half>(__half* p, float v) { *p = __float2half_rn(v); }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void store_out_dyn(void* base, int dtype, int64_t idx, float v) {
  if (dtype == FA_F32) reinterpret_cast<float*>(base)[idx] = v;
  else if (dtype == FA_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
}

#endif  // __CUDACC__

}  // namespace fa
