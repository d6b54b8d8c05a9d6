// Row-resident building block for the bandwidth kernels (softmax, RMSNorm, LayerNorm).
//
// One CTA owns one row (one Julia column: the contiguous, reduced dimension of length M).
// The row is read from HBM exactly once as 16-byte packets that stay in registers, the
// statistics are reduced with warp shuffles plus one shared-memory hop, and the result is
// written once.  THREADS x ITERS packets of 16 bytes cover the row; packets past the end
// are predicated off.
#pragma once
#include "common.cuh"

namespace tylo {

template <typename T, int THREADS, int ITERS> struct RowRegs {
  static constexpr int kVec = Elem<T>::kVec;
  static constexpr int kMaxElems = THREADS * ITERS * kVec;
  Pack<T> p[ITERS];

  __device__ __forceinline__ void load(const T* __restrict__ row, int nvec) {
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = i * THREADS + threadIdx.x;
      if (v < nvec) p[i].raw = ld_stream(row + (size_t)v * kVec);
      else p[i].raw = make_uint4(0, 0, 0, 0);
    }
  }
  __device__ __forceinline__ void store(T* __restrict__ row, int nvec) const {
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      const int v = i * THREADS + threadIdx.x;
      if (v < nvec) st_stream(row + (size_t)v * kVec, p[i].raw);
    }
  }
};

// Load one 16-byte packet of a small, reused vector (weights): default caching.
template <typename T> __device__ __forceinline__ Pack<T> ld_param(const T* p) {
  Pack<T> r;
  r.raw = *reinterpret_cast<const uint4*>(p);
  return r;
}

// Launch-shape table shared by the row kernels: (threads, packets per thread).
// Chosen so that each thread keeps 32-128 bytes of the row in flight.
struct RowShape { int threads, iters; };
inline bool pick_row_shape(int64_t nvec, int max_iters, RowShape* out) {
  static const RowShape table[] = {{32, 2}, {128, 2}, {256, 4}, {512, 8}, {1024, 8}};
  for (const RowShape& s : table) {
    if (s.iters <= max_iters && (int64_t)s.threads * s.iters >= nvec) { *out = s; return true; }
  }
  if (max_iters < 8 && nvec <= 1024 * (int64_t)max_iters) { *out = {1024, max_iters}; return true; }
  return false;
}

}  // namespace tylo
