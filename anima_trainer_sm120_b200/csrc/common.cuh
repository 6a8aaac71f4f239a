// Shared device/host helpers for the sm_100a kernels of this library.
//
// Conventions used by every translation unit here:
//   * entry points are extern "C", take raw device pointers + int64 sizes and a
//     cudaStream_t passed as void*, never allocate, never synchronise, and
//     return 0 or a negative ANIMA_E_* status (message via anima_last_error()).
//   * bf16 tensors travel as 16-bit words; all arithmetic is fp32 unless said.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/anima_b200.h"

namespace anima {

// ---- host-side error reporting -------------------------------------------------
void set_error(const char* fmt, ...);

#define ANIMA_REQUIRE(cond, code, ...)            \
  do {                                            \
    if (!(cond)) {                                \
      ::anima::set_error(__VA_ARGS__);            \
      return (code);                              \
    }                                             \
  } while (0)

#define ANIMA_CHECK_LAUNCH(what)                                                   \
  do {                                                                             \
    cudaError_t e__ = cudaGetLastError();                                          \
    if (e__ != cudaSuccess) {                                                      \
      ::anima::set_error("%s: launch failed: %s", what, cudaGetErrorString(e__));  \
      return ANIMA_E_CUDA;                                                         \
    }                                                                              \
  } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
__host__ __device__ static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Runs `f` (which returns a cudaError_t) once per CUDA device, with that device current, and remembers a
// success. cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a kernel's image in ONE device's context, so
// a process that uses several GPUs has to opt every kernel in on each of them.
struct PerDeviceOnce {
  std::mutex mu;
  bool done[64] = {};
};
template <class F>
cudaError_t per_device_once(PerDeviceOnce& st, F&& f) {
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  if (dev < 0 || dev >= 64) return f();
  std::lock_guard<std::mutex> lock(st.mu);
  if (st.done[dev]) return cudaSuccess;
  rc = f();
  if (rc == cudaSuccess) st.done[dev] = true;
  return rc;
}

// ---- device helpers ------------------------------------------------------------
#if defined(__CUDACC__)

struct __align__(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 raw;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}

// Streaming (evict-first) 16-byte global accesses: every tensor these kernels
// touch is larger than L2 and read or written exactly once.
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void stg_stream16(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum of `blocks` partial vectors of 64 floats (partial[b * 64 + e]) by one CTA of kFinalizeThreads threads:
// group q = thread / 64 adds its contiguous slice of the blocks in ascending order, then thread e < 64 adds
// the group sums in ascending order. The association is fixed, so the result is reproducible, and no thread
// walks more than blocks / 16 dependent loads. Returns the total in threads 0..63 (0 elsewhere).
constexpr int kFinalizeThreads = 1024;
__device__ __forceinline__ float sum_partials_64(const float* __restrict__ partial, int blocks) {
  __shared__ float group_sum[kFinalizeThreads / 64][64];
  const int e = threadIdx.x & 63, q = threadIdx.x >> 6;
  const int per = (blocks + kFinalizeThreads / 64 - 1) / (kFinalizeThreads / 64);
  const int b0 = q * per, b1 = min(blocks, b0 + per);
  float s = 0.f;
  for (int b = b0; b < b1; ++b) s += partial[b * 64 + e];
  group_sum[q][e] = s;
  __syncthreads();
  float total = 0.f;
  if (threadIdx.x < 64) {
#pragma unroll
    for (int g = 0; g < kFinalizeThreads / 64; ++g) total += group_sum[g][e];
  }
  return total;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

#endif  // __CUDACC__

}  // namespace anima
