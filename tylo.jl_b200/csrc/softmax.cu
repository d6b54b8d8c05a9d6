// Row softmax forward / backward for sm_100a: one read and one write of HBM per element
// (the reference's streaming kernel reads X twice, softmax.jl:6-33).
//
// A row of up to 8192 (16-bit) / 4096 (fp32) elements is held in the registers of one CTA.
// Longer rows are split across a thread-block cluster of 2, 4 or 8 CTAs whose partial
// (max, sum) pairs are exchanged through distributed shared memory, so that several
// part-rows are resident per SM and their load, exp and store phases overlap.
//
// exp is evaluated once per element: each thread first takes the max of its own elements,
// exponentiates against that, and the result is rescaled by exp2(m_thread - m_row) / sum
// — one extra exp per thread instead of one per element.
#include <cooperative_groups.h>

#include "rowwise.cuh"

namespace cg = cooperative_groups;

namespace tylo {

constexpr float kLog2e = 1.4426950408889634f;

// Combine a per-thread (max, sum-relative-to-that-max) pair over the CTA and, when CLUSTER > 1,
// over the cluster.  Returns the row max and the row sum relative to it.
template <int THREADS, bool CLUSTERED>
__device__ __forceinline__ void reduce_max_sum(float& m, float& s, float* smem /* >= 80 floats */) {
  // warp level
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const float mn = fmaxf(m, m2);
    s = (mn == -INFINITY) ? 0.f : s * exp2f(m - mn) + s2 * exp2f(m2 - mn);
    m = mn;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if constexpr (THREADS > 32) {
    if (lane == 0) { smem[warp] = m; smem[32 + warp] = s; }
    __syncthreads();
    m = lane < THREADS / 32 ? smem[lane] : -INFINITY;
    s = lane < THREADS / 32 ? smem[32 + lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m, m2);
      s = (mn == -INFINITY) ? 0.f : s * exp2f(m - mn) + s2 * exp2f(m2 - mn);
      m = mn;
    }
  }
  if constexpr (CLUSTERED) {
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();
    if (threadIdx.x == 0) { smem[64] = m; smem[65] = s; }
    cluster.sync();
    const unsigned n = cluster.num_blocks();
    float mr = -INFINITY, sr = 0.f;
    if (lane < (int)n) {
      const float* peer = cluster.map_shared_rank(smem, lane);
      mr = peer[64]; sr = peer[65];
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {  // cluster size <= 8
      const float m2 = __shfl_xor_sync(0xffffffffu, mr, o), s2 = __shfl_xor_sync(0xffffffffu, sr, o);
      const float mn = fmaxf(mr, m2);
      sr = (mn == -INFINITY) ? 0.f : sr * exp2f(mr - mn) + s2 * exp2f(m2 - mn);
      mr = mn;
    }
    m = __shfl_sync(0xffffffffu, mr, 0);
    s = __shfl_sync(0xffffffffu, sr, 0);
    cluster.sync();  // peers may exit (and release their shared memory) only after all reads
  } else if constexpr (THREADS > 32) {
    __syncthreads();
  }
}

template <int THREADS, bool CLUSTERED>
__device__ __forceinline__ float reduce_sum(float v, float* smem) {
  v = block_reduce<THREADS>(v, SumOp(), 0.f, smem);
  if constexpr (CLUSTERED) {
    cg::cluster_group cluster = cg::this_cluster();
    if (threadIdx.x == 0) smem[64] = v;
    cluster.sync();
    const unsigned n = cluster.num_blocks();
    const int lane = threadIdx.x & 31;
    float r = 0.f;
    if (lane < (int)n) r = cluster.map_shared_rank(smem, lane)[64];
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    v = __shfl_sync(0xffffffffu, r, 0);
    cluster.sync();
  }
  return v;
}

template <typename T, int THREADS, int ITERS, bool CLUSTERED>
__global__ void __launch_bounds__(THREADS)
softmax_fwd_kernel(T* __restrict__ Y, const T* __restrict__ X, int64_t M, int part_elems) {
  constexpr int VEC = Elem<T>::kVec;
  __shared__ float smem[80];
  unsigned csize = 1, crank = 0;
  if constexpr (CLUSTERED) {
    cg::cluster_group cluster = cg::this_cluster();
    csize = cluster.num_blocks(); crank = cluster.block_rank();
  }
  const size_t row = blockIdx.x / csize;
  const int64_t begin = (int64_t)crank * part_elems;
  int64_t len = M - begin; if (len > part_elems) len = part_elems; if (len < 0) len = 0;
  const int nvec = (int)(len / VEC);
  const T* x = X + row * M + begin;

  RowRegs<T, THREADS, ITERS> r;
  r.load(x, nvec);
  float e[ITERS][VEC];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    r.p[i].unpack(e[i]);
    if (i * THREADS + (int)threadIdx.x < nvec) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) m = fmaxf(m, e[i][j]);
    }
  }
  const float m_thread = m;
  const float mt = (m_thread == -INFINITY) ? 0.f : m_thread;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const bool live = i * THREADS + (int)threadIdx.x < nvec;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      e[i][j] = live ? exp2f((e[i][j] - mt) * kLog2e) : 0.f;
      s += e[i][j];
    }
  }
  m *= kLog2e;  // reductions run in log2 units
  reduce_max_sum<THREADS, CLUSTERED>(m, s, smem);
  // a row made only of -Inf yields zeros (nothing in the reference's tests pins that case)
  const float factor = (m_thread == -INFINITY) ? 0.f : exp2f(m_thread * kLog2e - m) / s;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
#pragma unroll
    for (int j = 0; j < VEC; ++j) e[i][j] *= factor;
    r.p[i].pack(e[i]);
  }
  r.store(Y + row * M + begin, nvec);
}

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Forward for 16-bit storage.  The row stays in registers in its packed 16-bit form (half the
// registers of an fp32 copy, so twice the bytes in flight per SM for the same occupancy) and exp is
// evaluated twice per element (once for the sum, once for the output) on the otherwise idle
// special-function unit; its approximate form is ample for a 16-bit result.
template <typename T, int THREADS, int ITERS>
__global__ void __launch_bounds__(THREADS)
softmax_fwd_packed_kernel(T* __restrict__ Y, const T* __restrict__ X, int64_t M) {
  constexpr int VEC = Elem<T>::kVec;
  __shared__ float smem[32];
  const int nvec = (int)(M / VEC);
  const size_t row = blockIdx.x;
  RowRegs<T, THREADS, ITERS> r;
  r.load(X + row * M, nvec);
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    if (i * THREADS + (int)threadIdx.x < nvec) {
      float f[VEC]; r.p[i].unpack(f);
#pragma unroll
      for (int j = 0; j < VEC; ++j) m = fmaxf(m, f[j]);
    }
  }
  m = block_reduce<THREADS>(m, MaxOp(), -INFINITY, smem);
  const float mo = (m == -INFINITY) ? 0.f : m * kLog2e;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    if (i * THREADS + (int)threadIdx.x < nvec) {
      float f[VEC]; r.p[i].unpack(f);
#pragma unroll
      for (int j = 0; j < VEC; ++j) s += ex2_fast(fmaf(f[j], kLog2e, -mo));
    }
  }
  s = block_reduce<THREADS>(s, SumOp(), 0.f, smem);
  const float inv = s > 0.f ? 1.f / s : 0.f;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    float f[VEC]; r.p[i].unpack(f);
#pragma unroll
    for (int j = 0; j < VEC; ++j) f[j] = ex2_fast(fmaf(f[j], kLog2e, -mo)) * inv;
    r.p[i].pack(f);
  }
  r.store(Y + row * M, nvec);
}

template <typename T, int THREADS, int ITERS, bool CLUSTERED>
__global__ void __launch_bounds__(THREADS)
softmax_bwd_kernel(T* __restrict__ dX, const T* __restrict__ dY, const T* __restrict__ Y, int64_t M,
                   int part_elems) {
  constexpr int VEC = Elem<T>::kVec;
  __shared__ float smem[80];
  unsigned csize = 1, crank = 0;
  if constexpr (CLUSTERED) {
    cg::cluster_group cluster = cg::this_cluster();
    csize = cluster.num_blocks(); crank = cluster.block_rank();
  }
  const size_t row = blockIdx.x / csize;
  const int64_t begin = (int64_t)crank * part_elems;
  int64_t len = M - begin; if (len > part_elems) len = part_elems; if (len < 0) len = 0;
  const int nvec = (int)(len / VEC);

  RowRegs<T, THREADS, ITERS> y, dy;
  y.load(Y + row * M + begin, nvec);
  dy.load(dY + row * M + begin, nvec);
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    float a[VEC], b[VEC];
    y.p[i].unpack(a); dy.p[i].unpack(b);
#pragma unroll
    for (int j = 0; j < VEC; ++j) dot += a[j] * b[j];
  }
  dot = reduce_sum<THREADS, CLUSTERED>(dot, smem);
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    float a[VEC], b[VEC];
    y.p[i].unpack(a); dy.p[i].unpack(b);
#pragma unroll
    for (int j = 0; j < VEC; ++j) a[j] = a[j] * (b[j] - dot);
    y.p[i].pack(a);
  }
  y.store(dX + row * M + begin, nvec);
}

// Long rows, backward: two passes over Y and dY instead of a register-resident row.  Pass 1 sums y * dy, pass 2
// reads both again — a row pair is 128 KB at 32,768 16-bit elements, a few hundred of them in flight fit L2 many
// times over, so the second read never reaches HBM — and writes dX.  No cluster, no row held in registers: a thread
// keeps eight 16-byte loads in flight and the CTA is free of the all-or-nothing scheduling of a cluster.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
softmax_bwd_twopass_kernel(T* __restrict__ dX, const T* __restrict__ dY, const T* __restrict__ Y, int64_t M) {
  constexpr int VEC = Elem<T>::kVec;
  __shared__ float smem[32];
  const size_t base = (size_t)blockIdx.x * M;
  const int nvec = (int)(M / VEC);
  const uint4* y4 = reinterpret_cast<const uint4*>(Y + base);
  const uint4* d4 = reinterpret_cast<const uint4*>(dY + base);
  float dot = 0.f;
  for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * THREADS) {
    Pack<T> y[4], d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * THREADS;
      y[u].raw = v < nvec ? __ldg(y4 + v) : make_uint4(0, 0, 0, 0);
      d[u].raw = v < nvec ? __ldg(d4 + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float a[VEC], b[VEC];
      y[u].unpack(a); d[u].unpack(b);
#pragma unroll
      for (int j = 0; j < VEC; ++j) dot = fmaf(a[j], b[j], dot);
    }
  }
  dot = block_reduce<THREADS>(dot, SumOp(), 0.f, smem);
  for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * THREADS) {
    Pack<T> y[4], d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * THREADS;
      y[u].raw = v < nvec ? __ldg(y4 + v) : make_uint4(0, 0, 0, 0);
      d[u].raw = v < nvec ? __ldg(d4 + v) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int v = v0 + u * THREADS;
      float a[VEC], b[VEC];
      y[u].unpack(a); d[u].unpack(b);
#pragma unroll
      for (int j = 0; j < VEC; ++j) a[j] = a[j] * (b[j] - dot);
      y[u].pack(a);
      if (v < nvec) st_stream(dX + base + (size_t)v * VEC, y[u].raw);
    }
  }
}

// Any M, any alignment: online max/sum pass, then a second pass that re-reads X (mostly from L2).
template <typename T>
__global__ void __launch_bounds__(256)
softmax_fwd_generic_kernel(T* __restrict__ Y, const T* __restrict__ X, int64_t M) {
  __shared__ float smem[80];
  const T* x = X + (size_t)blockIdx.x * M;
  float m = -INFINITY, s = 0.f;
  for (int64_t i = threadIdx.x; i < M; i += 256) {
    const float v = Elem<T>::to_f(x[i]) * kLog2e;
    const float mn = fmaxf(m, v);
    s = (mn == -INFINITY) ? 0.f : s * exp2f(m - mn) + exp2f(v - mn);
    m = mn;
  }
  reduce_max_sum<256, false>(m, s, smem);
  const float inv = 1.0f / s;
  for (int64_t i = threadIdx.x; i < M; i += 256)
    Y[(size_t)blockIdx.x * M + i] = Elem<T>::from_f(exp2f(Elem<T>::to_f(x[i]) * kLog2e - m) * inv);
}

template <typename T>
__global__ void __launch_bounds__(256)
softmax_bwd_generic_kernel(T* __restrict__ dX, const T* __restrict__ dY, const T* __restrict__ Y, int64_t M) {
  __shared__ float smem[32];
  const size_t base = (size_t)blockIdx.x * M;
  float dot = 0.f;
  for (int64_t i = threadIdx.x; i < M; i += 256) dot += Elem<T>::to_f(Y[base + i]) * Elem<T>::to_f(dY[base + i]);
  dot = block_reduce<256>(dot, SumOp(), 0.f, smem);
  for (int64_t i = threadIdx.x; i < M; i += 256)
    dX[base + i] = Elem<T>::from_f(Elem<T>::to_f(Y[base + i]) * (Elem<T>::to_f(dY[base + i]) - dot));
}

template <typename K, typename... Args>
static int32_t launch_clustered(K kernel, unsigned grid, unsigned threads, unsigned cluster, cudaStream_t st,
                                const char* what, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = 0; cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return TYLO_ERR_CUDA;
  }
  return TYLO_OK;
}

template <typename T, bool FWD>
static int32_t softmax_launch(void* out, const void* a, const void* b, int64_t M, int64_t N, cudaStream_t st) {
  constexpr int VEC = Elem<T>::kVec;
  constexpr int kPartVec = 256 * 4;  // packets per CTA in the clustered shape
  const char* what = FWD ? "softmax_fwd" : "softmax_bwd";
  if constexpr (FWD && VEC == 8) {
    if (M % VEC == 0 && M / VEC <= 512 * 16) {
      const int64_t nv = M / VEC;
#define TYLO_SMP(THREADS, ITERS)                                                                             \
  do {                                                                                                       \
    softmax_fwd_packed_kernel<T, THREADS, ITERS><<<(unsigned)N, THREADS, 0, st>>>((T*)out, (const T*)a, M);  \
    return check_launch(what);                                                                               \
  } while (0)
      if (nv <= 64) TYLO_SMP(32, 2);
      if (nv <= 256) TYLO_SMP(128, 2);
      if (nv <= 1024) TYLO_SMP(256, 4);
      if (nv <= 2048) TYLO_SMP(256, 8);
      if (nv <= 4096) TYLO_SMP(256, 16);
      TYLO_SMP(512, 16);
#undef TYLO_SMP
    }
  }
  if (M % VEC == 0) {
    const int64_t nvec = M / VEC;
#define TYLO_SM_LAUNCH(THREADS, ITERS)                                                                      \
  do {                                                                                                       \
    if constexpr (FWD) softmax_fwd_kernel<T, THREADS, ITERS, false><<<(unsigned)N, THREADS, 0, st>>>(          \
        (T*)out, (const T*)a, M, (int)M);                                                                    \
    else softmax_bwd_kernel<T, THREADS, ITERS, false><<<(unsigned)N, THREADS, 0, st>>>(                        \
        (T*)out, (const T*)a, (const T*)b, M, (int)M);                                                       \
    return check_launch(what);                                                                               \
  } while (0)
    if (nvec <= 64) TYLO_SM_LAUNCH(32, 2);
    if (nvec <= 256) TYLO_SM_LAUNCH(128, 2);
    if (nvec <= kPartVec) TYLO_SM_LAUNCH(256, 4);
#undef TYLO_SM_LAUNCH
    if constexpr (!FWD) {
      // rows too long for one CTA's registers: the two-pass form (4,952 GB/s with the clustered register-resident
      // form on 4096 x 32768 bf16, 6,225 with this one at 1,024 threads; 5,317 at 512 and 4,042 at 256 threads)
      if (nvec > kPartVec) {
        softmax_bwd_twopass_kernel<T, 1024><<<(unsigned)N, 1024, 0, st>>>((T*)out, (const T*)a, (const T*)b, M);
        return check_launch(what);
      }
    }
    if (nvec <= 8 * kPartVec && N * 8 <= 0x7fffffffLL) {
      unsigned c = 2;
      while ((int64_t)c * kPartVec < nvec) c *= 2;
      // even split, rounded up to whole packets
      const int part = (int)(((nvec + c - 1) / c) * VEC);
      if constexpr (FWD)
        return launch_clustered(softmax_fwd_kernel<T, 256, 4, true>, (unsigned)(N * c), 256, c, st, what,
                                (T*)out, (const T*)a, M, part);
      else
        return launch_clustered(softmax_bwd_kernel<T, 256, 4, true>, (unsigned)(N * c), 256, c, st, what,
                                (T*)out, (const T*)a, (const T*)b, M, part);
    }
  }
  if constexpr (FWD) softmax_fwd_generic_kernel<T><<<(unsigned)N, 256, 0, st>>>((T*)out, (const T*)a, M);
  else softmax_bwd_generic_kernel<T><<<(unsigned)N, 256, 0, st>>>((T*)out, (const T*)a, (const T*)b, M);
  return check_launch(what);
}

}  // namespace tylo

using namespace tylo;

extern "C" int32_t tylo_b200_softmax_fwd(void* Y, const void* X, int64_t M, int64_t N, int32_t dtype,
                                         tylo_stream_t stream) {
  TYLO_REQUIRE(Y && X, TYLO_ERR_INVALID_ARGUMENT, "softmax_fwd: Y and X must be non-null");
  TYLO_REQUIRE(M > 0 && N > 0, TYLO_ERR_INVALID_ARGUMENT, "softmax_fwd: extents must be positive (M=%lld, N=%lld)",
               (long long)M, (long long)N);
  TYLO_REQUIRE(N <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED, "softmax_fwd: N above 2^31-1 is not supported");
  TYLO_REQUIRE(aligned16(Y) && aligned16(X), TYLO_ERR_MISALIGNED, "softmax_fwd: pointers must be 16-byte aligned");
  TYLO_DISPATCH_DTYPE(dtype, T, return (softmax_launch<T, true>(Y, X, nullptr, M, N, (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_softmax_bwd(void* dX, const void* dY, const void* Y, int64_t M, int64_t N,
                                         int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(dX && dY && Y, TYLO_ERR_INVALID_ARGUMENT, "softmax_bwd: dX, dY and Y must be non-null");
  TYLO_REQUIRE(M > 0 && N > 0, TYLO_ERR_INVALID_ARGUMENT, "softmax_bwd: extents must be positive (M=%lld, N=%lld)",
               (long long)M, (long long)N);
  TYLO_REQUIRE(N <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED, "softmax_bwd: N above 2^31-1 is not supported");
  TYLO_REQUIRE(aligned16(dX) && aligned16(dY) && aligned16(Y), TYLO_ERR_MISALIGNED,
               "softmax_bwd: pointers must be 16-byte aligned");
  // argument order of the kernel: (dX, dY, Y)
  TYLO_DISPATCH_DTYPE(dtype, T, return (softmax_launch<T, false>(dX, dY, Y, M, N, (cudaStream_t)stream)));
  return TYLO_OK;
}
