// Shared helpers for the sso_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <string>

#include "../../include/sso_b200.h"

namespace sso {

// Last error text, per host thread (backward hooks call in from autograd's thread).
extern thread_local std::string g_last_error;
// Number of kernels this library has launched (all threads); read with sso_launch_count().
extern unsigned long long g_launches;

inline int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
inline int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define SSO_CHECK_ARG(cond, ...)                      \
  do {                                                \
    if (!(cond)) return ::sso::fail(-1, __VA_ARGS__); \
  } while (0)

#define SSO_CUDA_OK(expr)                                                                    \
  do {                                                                                       \
    cudaError_t e__ = (expr);                                                                \
    if (e__ != cudaSuccess)                                                                  \
      return ::sso::fail(-2, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                         __LINE__);                                                          \
  } while (0)

#define SSO_LAUNCH_OK(name)                                                                 \
  do {                                                                                      \
    __atomic_add_fetch(&::sso::g_launches, 1ull, __ATOMIC_RELAXED);                         \
    cudaError_t e__ = cudaGetLastError();                                                   \
    if (e__ != cudaSuccess)                                                                 \
      return ::sso::fail(-3, "launch of %s failed: %s", name, cudaGetErrorString(e__));     \
  } while (0)

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) applies to the device that is current when it is
// called: remember per (kernel, device) what has been set (api.cu; thread safe).
int ensure_dynamic_smem(const void* kernel, int bytes);
#define SSO_ENSURE_SMEM(kernel, bytes)                                                   \
  do {                                                                                   \
    const int rc__ = ::sso::ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), (int)(bytes)); \
    if (rc__) return rc__;                                                               \
  } while (0)

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Lower-triangle tile index t -> (bi, bj) with bi >= bj, t = bi*(bi+1)/2 + bj.
__device__ __forceinline__ void tri_decode(int t, int& bi, int& bj) {
  int r = (int)((sqrtf(8.0f * (float)t + 1.0f) - 1.0f) * 0.5f);
  while (r * (r + 1) / 2 > t) --r;
  while ((r + 1) * (r + 2) / 2 <= t) ++r;
  bi = r;
  bj = t - r * (r + 1) / 2;
}

// ------------------------------------------------------------------------------------------
// SIMT tile core: 256 threads compute a (16*MT) x (16*MT) tile; operands are staged in shared
// memory as [32 k][16*MT] fp32 with a 16-byte-granular XOR swizzle on the column index so that
// both the transposing stores of the loaders and the float4 reads below are conflict free.
// ------------------------------------------------------------------------------------------
constexpr int KT = 32;  // contraction depth of one shared-memory stage

__device__ __forceinline__ int swz(int k, int col) { return col ^ ((k & 7) << 2); }

template <int MT>
struct TileCore {
  static constexpr int TILE = 16 * MT;
  static constexpr int NV = MT / 4;  // float4 groups per thread per operand

  // acc[i][j]: i indexes this thread's MT rows, j its MT columns.
  // Rows owned: for g in [0,NV): g*64 + ty*4 + q; columns alike with tx.
  __device__ __forceinline__ static void compute(const float* __restrict__ As,
                                                 const float* __restrict__ Bs, int ty, int tx,
                                                 float (&acc)[MT][MT]) {
#pragma unroll 8
    for (int k = 0; k < KT; ++k) {
      float a[MT], b[MT];
#pragma unroll
      for (int g = 0; g < NV; ++g) {
        const float4 va = *reinterpret_cast<const float4*>(As + k * TILE + swz(k, g * 64 + ty * 4));
        const float4 vb = *reinterpret_cast<const float4*>(Bs + k * TILE + swz(k, g * 64 + tx * 4));
        a[g * 4 + 0] = va.x; a[g * 4 + 1] = va.y; a[g * 4 + 2] = va.z; a[g * 4 + 3] = va.w;
        b[g * 4 + 0] = vb.x; b[g * 4 + 1] = vb.y; b[g * 4 + 2] = vb.z; b[g * 4 + 3] = vb.w;
      }
#pragma unroll
      for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < MT; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }
  __device__ __forceinline__ static int row_of(int ty, int i) { return (i / 4) * 64 + ty * 4 + (i & 3); }
  __device__ __forceinline__ static int col_of(int tx, int j) { return (j / 4) * 64 + tx * 4 + (j & 3); }
};

}  // namespace sso
