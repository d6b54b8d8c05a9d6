// Shared host/device helpers for libtylo_b200: status plumbing, dtype dispatch,
// 16-byte vector access and warp/block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/tylo_b200.h"

namespace tylo {

// ---- status ---------------------------------------------------------------------------------
void set_error(const char* fmt, ...);  // defined in api.cu (thread-local buffer)

#define TYLO_REQUIRE(cond, code, ...)        \
  do {                                       \
    if (!(cond)) {                           \
      ::tylo::set_error(__VA_ARGS__);        \
      return (code);                         \
    }                                        \
  } while (0)

#define TYLO_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      ::tylo::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));               \
      return TYLO_ERR_CUDA;                                                             \
    }                                                                                   \
  } while (0)

inline int32_t check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return TYLO_ERR_CUDA;
  }
  return TYLO_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// ---- dtype traits -----------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kVec = 4;  // elements per 16 bytes
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

// 16-byte packet of T, unpacked to / packed from fp32.
template <typename T> struct Pack {
  static constexpr int kVec = Elem<T>::kVec;
  uint4 raw;
  __device__ __forceinline__ void unpack(float (&f)[Elem<T>::kVec]) const;
  __device__ __forceinline__ void pack(const float (&f)[Elem<T>::kVec]);
};
template <> __device__ __forceinline__ void Pack<float>::unpack(float (&f)[4]) const {
  f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
  f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void Pack<float>::pack(const float (&f)[4]) {
  raw.x = __float_as_uint(f[0]); raw.y = __float_as_uint(f[1]);
  raw.z = __float_as_uint(f[2]); raw.w = __float_as_uint(f[3]);
}
template <> __device__ __forceinline__ void Pack<__nv_bfloat16>::unpack(float (&f)[8]) const {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {  // bf16 -> fp32 is a 16-bit shift
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void Pack<__nv_bfloat16>::pack(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&p);
  }
  raw = make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ void Pack<__half>::unpack(float (&f)[8]) const {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = p.x; f[2 * i + 1] = p.y;
  }
}
template <> __device__ __forceinline__ void Pack<__half>::pack(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 p = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&p);
  }
  raw = make_uint4(w[0], w[1], w[2], w[3]);
}

// Streaming 16-byte global access: data touched once, keep it out of L1.
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- reductions -----------------------------------------------------------------------------
struct SumOp { __device__ __forceinline__ float operator()(float a, float b) const { return a + b; } };
struct MaxOp { __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); } };

template <typename Op> __device__ __forceinline__ float warp_reduce(float v, Op op) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// All threads of the block receive the result.  `scratch` holds >= 32 floats and may be
// reused for the next reduction only after the trailing barrier (included).
template <int THREADS, typename Op>
__device__ __forceinline__ float block_reduce(float v, Op op, float identity, float* scratch) {
  v = warp_reduce(v, op);
  if constexpr (THREADS == 32) return v;
  constexpr int kWarps = THREADS / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < kWarps ? scratch[lane] : identity;
  r = warp_reduce(r, op);
  __syncthreads();
  return r;
}

// dtype dispatch for host code
#define TYLO_DISPATCH_DTYPE(dtype, T, ...)                                   \
  switch (dtype) {                                                           \
    case TYLO_F32: { using T = float; __VA_ARGS__; break; }                  \
    case TYLO_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }         \
    case TYLO_F16: { using T = __half; __VA_ARGS__; break; }                 \
    default:                                                                 \
      ::tylo::set_error("unknown dtype %d", (int)(dtype));                   \
      return TYLO_ERR_INVALID_ARGUMENT;                                      \
  }

}  // namespace tylo
