// Shared device/host helpers for the kvq_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/kvq_b200.h"

namespace kvq {

// ---- host: error reporting -------------------------------------------------------------------
void set_error(const char* fmt, ...);  // stores a message for kvq_last_error() on this thread

#define KVQ_REQUIRE(cond, ...)                \
  do {                                        \
    if (!(cond)) {                            \
      kvq::set_error(__VA_ARGS__);            \
      return KVQ_ERR_INVALID_ARGUMENT;        \
    }                                         \
  } while (0)

#define KVQ_CUDA(call)                                                                  \
  do {                                                                                  \
    cudaError_t e_ = (call);                                                            \
    if (e_ != cudaSuccess) {                                                            \
      kvq::set_error("%s failed: %s", #call, cudaGetErrorString(e_));                   \
      return KVQ_ERR_CUDA;                                                              \
    }                                                                                   \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- device: exact quantization primitives ---------------------------------------------------
// clamp(round_half_even(x), -127, 127): -128 is never produced.
__device__ __forceinline__ int sat127(float x) { return max(-127, min(127, __float2int_rn(x))); }

// IEEE fp32 division then round/clamp; matches torch.clamp(torch.round(x / s), -127, 127).
__device__ __forceinline__ int quant1(float x, float s) { return sat127(__fdiv_rn(x, s)); }

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  return (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | (static_cast<uint32_t>(d) << 24);
}

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Streaming 16-byte global accesses for data touched exactly once.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

}  // namespace kvq
