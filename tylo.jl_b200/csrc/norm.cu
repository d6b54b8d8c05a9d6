// RMSNorm and LayerNorm, forward and backward, for sm_100a.
//
// Forward: one pass over HBM (read X once, write Y once); the row lives in registers, the
// statistics are fp32.  LayerNorm's variance is the centred second moment computed from the
// registers, so it has the accuracy of the reference's three-pass kernel without its two
// extra reads (layer_norm.jl:6-46 reads X three times, rms_norm.jl:6-32 twice).
//
// Backward: `n_groups` CTAs stride over the rows.  Each keeps its partial dW (and dB) for the
// columns it owns in registers and writes one row of the fp32 partial buffer at the end; a
// second kernel sums the partial rows.  No locks, no atomics, deterministic
// (the reference serialises the groups on a global spin-lock: rms_norm.jl:68-78,
// layer_norm.jl:102-116).
#include "rowwise.cuh"
#include "sm100_ptx.cuh"


namespace tylo {

#define TYLO_ROW_DISPATCH(shape, ...)                                                          \
  do {                                                                                         \
    if ((shape).threads == 32 && (shape).iters == 2) { constexpr int THREADS = 32, ITERS = 2; __VA_ARGS__; }          \
    else if ((shape).threads == 128 && (shape).iters == 2) { constexpr int THREADS = 128, ITERS = 2; __VA_ARGS__; }   \
    else if ((shape).threads == 256 && (shape).iters == 4) { constexpr int THREADS = 256, ITERS = 4; __VA_ARGS__; }   \
    else if ((shape).threads == 512 && (shape).iters == 8) { constexpr int THREADS = 512, ITERS = 8; __VA_ARGS__; }   \
    else if ((shape).threads == 1024 && (shape).iters == 8) { constexpr int THREADS = 1024, ITERS = 8; __VA_ARGS__; } \
    else { constexpr int THREADS = 1024, ITERS = 4; __VA_ARGS__; }                                                    \
  } while (0)

// Merge of two (count, mean, M2) partial statistics.
__device__ __forceinline__ void welford_merge(float& n, float& mu, float& m2, float nb, float mub, float m2b) {
  const float nt = n + nb;
  if (nt > 0.f) {
    const float d = mub - mu, f = nb / nt;
    mu += d * f;
    m2 += m2b + d * d * n * f;
  }
  n = nt;
}
// Same for partial statistics of EQUAL counts (every thread holds the same number of elements, the
// common case): no division, `half_n` = elements per side / 2 ... passed as the per-side count.
template <int THREADS>
__device__ __forceinline__ void welford_block_equal(float per_thread, float& mu, float& m2, float* scratch) {
  float n = per_thread;   // elements per side at this level
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float mub = __shfl_xor_sync(0xffffffffu, mu, o), m2b = __shfl_xor_sync(0xffffffffu, m2, o);
    const float d = mub - mu;
    mu = 0.5f * (mu + mub);
    m2 = m2 + m2b + d * d * (0.5f * n);
    n *= 2.f;
  }
  if constexpr (THREADS > 32) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { scratch[warp] = mu; scratch[32 + warp] = m2; }
    __syncthreads();
    mu = scratch[lane & (kWarps - 1)];
    m2 = scratch[32 + (lane & (kWarps - 1))];
#pragma unroll
    for (int o = 1; o < kWarps; o <<= 1) {
      const float mub = __shfl_xor_sync(0xffffffffu, mu, o), m2b = __shfl_xor_sync(0xffffffffu, m2, o);
      const float d = mub - mu;
      mu = 0.5f * (mu + mub);
      m2 = m2 + m2b + d * d * (0.5f * n);
      n *= 2.f;
    }
  }
}

// All threads receive the block-wide (count, mean, M2).  `scratch` holds 96 floats.
template <int THREADS>
__device__ __forceinline__ void welford_block(float& n, float& mu, float& m2, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float nb = __shfl_xor_sync(0xffffffffu, n, o), mub = __shfl_xor_sync(0xffffffffu, mu, o),
                m2b = __shfl_xor_sync(0xffffffffu, m2, o);
    welford_merge(n, mu, m2, nb, mub, m2b);
  }
  if constexpr (THREADS > 32) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { scratch[warp] = n; scratch[32 + warp] = mu; scratch[64 + warp] = m2; }
    __syncthreads();
    n = lane < kWarps ? scratch[lane] : 0.f;
    mu = lane < kWarps ? scratch[32 + lane] : 0.f;
    m2 = lane < kWarps ? scratch[64 + lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float nb = __shfl_xor_sync(0xffffffffu, n, o), mub = __shfl_xor_sync(0xffffffffu, mu, o),
                  m2b = __shfl_xor_sync(0xffffffffu, m2, o);
      welford_merge(n, mu, m2, nb, mub, m2b);
    }
  }
  // the merge is not bit-commutative: every thread takes lane 0's result
  n = __shfl_sync(0xffffffffu, n, 0); mu = __shfl_sync(0xffffffffu, mu, 0); m2 = __shfl_sync(0xffffffffu, m2, 0);
}

// ------------------------------------------------------------------------------------------------
// forward, row in registers
// ------------------------------------------------------------------------------------------------
template <typename T, int THREADS, int ITERS, bool LAYER>
__global__ void __launch_bounds__(THREADS)
norm_fwd_kernel(T* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ W,
                const T* __restrict__ Bias, float* __restrict__ Mean, float* __restrict__ Rstd,
                int M, float eps, float offset) {
  constexpr int VEC = Elem<T>::kVec;
  __shared__ float red[32];
  __shared__ float wred[LAYER ? 96 : 1];
  const int nvec = M / VEC;
  const size_t row = blockIdx.x;
  RowRegs<T, THREADS, ITERS> x;
  x.load(X + row * M, nvec);

  const float inv_m = 1.0f / (float)M;
  float mean = 0.f;
  float ss = 0.f;
  if constexpr (LAYER) {
    // Per-thread mean and centred second moment from the registers, then ONE reduction round that
    // merges (count, mean, M2) triples (Chan et al.): centred accuracy without a second barrier.
    float cnt = 0.f, s = 0.f;
    // two elements per instruction (packed fp32 pairs): the kernel is close enough to the issue limit
    // for the instruction count to show in its bandwidth
    uint64_t s2 = 0ull;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      if (i * THREADS + (int)threadIdx.x < nvec) {
        float f[VEC]; x.p[i].unpack(f);
#pragma unroll
        for (int j = 0; j < VEC; j += 2) s2 = sm100::add_f32x2(s2, sm100::pack_f32x2(f[j], f[j + 1]));
        cnt += (float)VEC;
      }
    }
    { float a, b; sm100::unpack_f32x2(s2, a, b); s = a + b; }
    float mu = cnt > 0.f ? s / cnt : 0.f, m2 = 0.f;
    const uint64_t nmu2 = sm100::pack_f32x2(-mu, -mu);
    uint64_t q2 = 0ull;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      if (i * THREADS + (int)threadIdx.x < nvec) {
        float f[VEC]; x.p[i].unpack(f);
#pragma unroll
        for (int j = 0; j < VEC; j += 2) {
          const uint64_t c2 = sm100::add_f32x2(sm100::pack_f32x2(f[j], f[j + 1]), nmu2);
          q2 = sm100::fma_f32x2(c2, c2, q2);
        }
      }
    }
    { float a, b; sm100::unpack_f32x2(q2, a, b); m2 = a + b; }
    if (nvec == THREADS * ITERS) welford_block_equal<THREADS>((float)(ITERS * VEC), mu, m2, wred);
    else welford_block<THREADS>(cnt, mu, m2, wred);
    mean = mu; ss = m2;
  } else {
    uint64_t q2 = 0ull;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      float f[VEC]; x.p[i].unpack(f);     // packets past the end are zero
#pragma unroll
      for (int j = 0; j < VEC; j += 2) {
        const uint64_t v2 = sm100::pack_f32x2(f[j], f[j + 1]);
        q2 = sm100::fma_f32x2(v2, v2, q2);
      }
    }
    { float a, b; sm100::unpack_f32x2(q2, a, b); ss = a + b; }
    ss = block_reduce<THREADS>(ss, SumOp(), 0.f, red);
  }
  const float rstd = 1.0f / sqrtf(ss * inv_m + eps);
  if (threadIdx.x == 0) {
    if (Rstd) Rstd[row] = rstd;
    if (LAYER && Mean) Mean[row] = mean;
  }
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int v = i * THREADS + threadIdx.x;
    if (v < nvec) {
      float f[VEC], w[VEC], b[VEC];
      x.p[i].unpack(f);
      ld_param(W + (size_t)v * VEC).unpack(w);
      if constexpr (LAYER) ld_param(Bias + (size_t)v * VEC).unpack(b);
      if constexpr (LAYER) {
        // ((x - mean) rstd) w + b on pairs: (x + (-mean)) * (rstd w) + b
        const uint64_t nmean2 = sm100::pack_f32x2(-mean, -mean), rstd2 = sm100::pack_f32x2(rstd, rstd);
#pragma unroll
        for (int j = 0; j < VEC; j += 2) {
          const uint64_t c2 = sm100::add_f32x2(sm100::pack_f32x2(f[j], f[j + 1]), nmean2);
          const uint64_t a2 = sm100::mul_f32x2(sm100::pack_f32x2(w[j], w[j + 1]), rstd2);
          sm100::unpack_f32x2(sm100::fma_f32x2(c2, a2, sm100::pack_f32x2(b[j], b[j + 1])), f[j], f[j + 1]);
        }
      } else {
        const uint64_t rstd2 = sm100::pack_f32x2(rstd, rstd), off2 = sm100::pack_f32x2(offset, offset);
#pragma unroll
        for (int j = 0; j < VEC; j += 2) {
          const uint64_t a2 = sm100::mul_f32x2(sm100::add_f32x2(sm100::pack_f32x2(w[j], w[j + 1]), off2), rstd2);
          sm100::unpack_f32x2(sm100::mul_f32x2(sm100::pack_f32x2(f[j], f[j + 1]), a2), f[j], f[j + 1]);
        }
      }
      x.p[i].pack(f);
    }
  }
  x.store(Y + row * M, nvec);
}

// forward, any M and any row alignment: scalar accesses, X re-read from L2.
template <typename T, bool LAYER>
__global__ void __launch_bounds__(256)
norm_fwd_generic_kernel(T* __restrict__ Y, const T* __restrict__ X, const T* __restrict__ W,
                        const T* __restrict__ Bias, float* __restrict__ Mean,
                        float* __restrict__ Rstd, int64_t M, float eps, float offset) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const T* x = X + row * M;
  const float inv_m = 1.0f / (float)M;
  float mean = 0.f;
  if constexpr (LAYER) {
    float s = 0.f;
    for (int64_t i = threadIdx.x; i < M; i += 256) s += Elem<T>::to_f(x[i]);
    mean = block_reduce<256>(s, SumOp(), 0.f, red) * inv_m;
  }
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < M; i += 256) {
    const float c = Elem<T>::to_f(x[i]) - mean;
    ss += c * c;
  }
  ss = block_reduce<256>(ss, SumOp(), 0.f, red);
  const float rstd = 1.0f / sqrtf(ss * inv_m + eps);
  if (threadIdx.x == 0) {
    if (Rstd) Rstd[row] = rstd;
    if (LAYER && Mean) Mean[row] = mean;
  }
  for (int64_t i = threadIdx.x; i < M; i += 256) {
    const float f = Elem<T>::to_f(x[i]);
    float y;
    if constexpr (LAYER) y = (f - mean) * rstd * Elem<T>::to_f(W[i]) + Elem<T>::to_f(Bias[i]);
    else y = f * rstd * (Elem<T>::to_f(W[i]) + offset);
    Y[row * M + i] = Elem<T>::from_f(y);
  }
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
template <typename T, int THREADS, int ITERS, bool LAYER>
__global__ void __launch_bounds__(THREADS)
norm_bwd_kernel(T* __restrict__ dX, float* __restrict__ dWp, float* __restrict__ dBp,
                const T* __restrict__ dY, const T* __restrict__ X, const T* __restrict__ W,
                const float* __restrict__ Mean, const float* __restrict__ Rstd,
                int M, int64_t N, float offset) {
  constexpr int VEC = Elem<T>::kVec;
  __shared__ float red[64];
  const int nvec = M / VEC;
  const float inv_m = 1.0f / (float)M;

  float g[ITERS][VEC];       // w (+offset) for the columns this thread owns
  float dw[ITERS][VEC], db[LAYER ? ITERS : 1][VEC];
#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int v = i * THREADS + threadIdx.x;
    if (v < nvec) ld_param(W + (size_t)v * VEC).unpack(g[i]);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      if (v >= nvec) g[i][j] = 0.f;
      if constexpr (!LAYER) g[i][j] += offset;
      dw[i][j] = 0.f;
      if constexpr (LAYER) db[i][j] = 0.f;
    }
  }

  for (int64_t row = blockIdx.x; row < N; row += gridDim.x) {
    RowRegs<T, THREADS, ITERS> x, dy;
    x.load(X + row * M, nvec);
    dy.load(dY + row * M, nvec);
    const float rstd = Rstd[row];
    const float mean = LAYER ? Mean[row] : 0.f;
    // c1 = mean(xhat * g*dy), c2 = mean(g*dy) (LayerNorm only)
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      float xf[VEC], df[VEC];
      x.p[i].unpack(xf); dy.p[i].unpack(df);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float xhat = (xf[j] - mean) * rstd;   // zero packets contribute g = 0
        const float gd = g[i][j] * df[j];
        s1 += xhat * gd;
        if constexpr (LAYER) s2 += gd;
      }
    }
    // two sums through one reduction round
    s1 = warp_reduce(s1, SumOp());
    if constexpr (LAYER) s2 = warp_reduce(s2, SumOp());
    if constexpr (THREADS > 32) {
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      if (lane == 0) { red[warp] = s1; red[32 + warp] = s2; }
      __syncthreads();
      float a = lane < THREADS / 32 ? red[lane] : 0.f;
      float b = lane < THREADS / 32 ? red[32 + lane] : 0.f;
      s1 = warp_reduce(a, SumOp());
      if constexpr (LAYER) s2 = warp_reduce(b, SumOp());
      __syncthreads();
    }
    const float c1 = s1 * inv_m, c2 = s2 * inv_m;
#pragma unroll
    for (int i = 0; i < ITERS; ++i) {
      float xf[VEC], df[VEC], o[VEC];
      x.p[i].unpack(xf); dy.p[i].unpack(df);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float xhat = (xf[j] - mean) * rstd;
        const float gd = g[i][j] * df[j];
        // RMS: rstd*(dy*g - rstd^2*dd*x) with xhat = x*rstd, c1 = rstd*dd  (test/norm.jl:78-87)
        // LN : (g*dy - (xhat*c1 + c2))*rstd                                  (test/norm.jl:90-102)
        o[j] = (gd - (xhat * c1 + c2)) * rstd;
        dw[i][j] += df[j] * xhat;
        if constexpr (LAYER) db[i][j] += df[j];
      }
      x.p[i].pack(o);
    }
    x.store(dX + row * M, nvec);
  }

#pragma unroll
  for (int i = 0; i < ITERS; ++i) {
    const int v = i * THREADS + threadIdx.x;
    if (v < nvec) {
      float4* pw = reinterpret_cast<float4*>(dWp + (size_t)blockIdx.x * M + (size_t)v * VEC);
#pragma unroll
      for (int j = 0; j < VEC; j += 4) pw[j / 4] = make_float4(dw[i][j], dw[i][j + 1], dw[i][j + 2], dw[i][j + 3]);
      if constexpr (LAYER) {
        float4* pb = reinterpret_cast<float4*>(dBp + (size_t)blockIdx.x * M + (size_t)v * VEC);
#pragma unroll
        for (int j = 0; j < VEC; j += 4) pb[j / 4] = make_float4(db[i][j], db[i][j + 1], db[i][j + 2], db[i][j + 3]);
      }
    }
  }
}

// backward, streaming form for rows of exactly THREADS packets (one 16-byte packet of X and of dY per
// thread): the per-thread state is a handful of registers, so the packets of the next TWO rows are
// already in flight while the current row is reduced — the HBM stream never waits for a reduction.
// One barrier per row (the reduction scratch is double-buffered).
template <typename T, int THREADS, bool LAYER>
__global__ void __launch_bounds__(THREADS)
norm_bwd_stream_kernel(T* __restrict__ dX, float* __restrict__ dWp, float* __restrict__ dBp,
                       const T* __restrict__ dY, const T* __restrict__ X, const T* __restrict__ W,
                       const float* __restrict__ Mean, const float* __restrict__ Rstd,
                       int M, int64_t N, float offset) {
  constexpr int VEC = Elem<T>::kVec;
  constexpr int kWarps = THREADS / 32;
  __shared__ float red[2][64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t col = (size_t)threadIdx.x * VEC;
  const float inv_m = 1.0f / (float)M;
  float g[VEC], dw[VEC], db[VEC];
  ld_param(W + col).unpack(g);
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    if constexpr (!LAYER) g[j] += offset;
    dw[j] = 0.f; db[j] = 0.f;
  }
  const int64_t stride = gridDim.x;
  Pack<T> x0, d0, x1, d1, x2, d2;
  float r0 = 0.f, r1 = 0.f, r2 = 0.f, m0 = 0.f, m1 = 0.f, m2 = 0.f;
  auto fetch = [&](int64_t r, Pack<T>& x, Pack<T>& d, float& rs, float& mn) {
    if (r < N) {
      x.raw = ld_stream(X + r * M + col); d.raw = ld_stream(dY + r * M + col);
      rs = Rstd[r];
      mn = LAYER ? Mean[r] : 0.f;
    }
  };
  int64_t row = blockIdx.x;
  // rows in flight behind the current one: two for RMSNorm, one for LayerNorm (its extra accumulators
  // and statistics would otherwise push the 1024-thread CTA past 64 registers per thread)
  fetch(row, x0, d0, r0, m0);
  if constexpr (!LAYER) fetch(row + stride, x1, d1, r1, m1);
  for (int par = 0; row < N; row += stride, par ^= 1) {
    if constexpr (LAYER) fetch(row + stride, x1, d1, r1, m1);
    else fetch(row + 2 * stride, x2, d2, r2, m2);
    float s1 = 0.f, s2 = 0.f;
    const uint64_t nm2 = sm100::pack_f32x2(-m0, -m0), r2p = sm100::pack_f32x2(r0, r0);
    {
      // packed fp32 pairs: xhat = (x - mean) rstd, gd = g dy, s1 += xhat gd, s2 += gd
      float xf[VEC], df[VEC];
      x0.unpack(xf); d0.unpack(df);
      uint64_t a1 = 0ull, a2 = 0ull;
#pragma unroll
      for (int j = 0; j < VEC; j += 2) {
        const uint64_t gd2 = sm100::mul_f32x2(sm100::pack_f32x2(g[j], g[j + 1]), sm100::pack_f32x2(df[j], df[j + 1]));
        const uint64_t xh2 = sm100::mul_f32x2(sm100::add_f32x2(sm100::pack_f32x2(xf[j], xf[j + 1]), nm2), r2p);
        a1 = sm100::fma_f32x2(xh2, gd2, a1);
        if constexpr (LAYER) a2 = sm100::add_f32x2(a2, gd2);
      }
      float lo, hi;
      sm100::unpack_f32x2(a1, lo, hi); s1 = lo + hi;
      if constexpr (LAYER) { sm100::unpack_f32x2(a2, lo, hi); s2 = lo + hi; }
    }
    s1 = warp_reduce(s1, SumOp());
    if constexpr (LAYER) s2 = warp_reduce(s2, SumOp());
    if (lane == 0) { red[par][warp] = s1; red[par][32 + warp] = s2; }
    __syncthreads();
    s1 = warp_reduce(lane < kWarps ? red[par][lane] : 0.f, SumOp());
    if constexpr (LAYER) s2 = warp_reduce(lane < kWarps ? red[par][32 + lane] : 0.f, SumOp());
    const float c1 = s1 * inv_m, c2 = LAYER ? s2 * inv_m : 0.f;
    // the packets are unpacked again rather than kept as fp32 across the barrier (registers)
    float xf[VEC], df[VEC], o[VEC];
    x0.unpack(xf); d0.unpack(df);
    const uint64_t nc1 = sm100::pack_f32x2(-c1, -c1), nc2 = sm100::pack_f32x2(-c2, -c2);
#pragma unroll
    for (int j = 0; j < VEC; j += 2) {
      // same formulas as norm_bwd_kernel, two columns per instruction:
      // dx = (g dy - (xhat c1 + c2)) rstd,  dW += dy xhat,  dB += dy
      const uint64_t df2 = sm100::pack_f32x2(df[j], df[j + 1]);
      const uint64_t xh2 = sm100::mul_f32x2(sm100::add_f32x2(sm100::pack_f32x2(xf[j], xf[j + 1]), nm2), r2p);
      const uint64_t t2 = sm100::fma_f32x2(xh2, nc1, nc2);
      const uint64_t o2 = sm100::mul_f32x2(sm100::fma_f32x2(sm100::pack_f32x2(g[j], g[j + 1]), df2, t2), r2p);
      sm100::unpack_f32x2(o2, o[j], o[j + 1]);
      const uint64_t w2 = sm100::fma_f32x2(df2, xh2, sm100::pack_f32x2(dw[j], dw[j + 1]));
      sm100::unpack_f32x2(w2, dw[j], dw[j + 1]);
      if constexpr (LAYER) {
        const uint64_t b2 = sm100::add_f32x2(sm100::pack_f32x2(db[j], db[j + 1]), df2);
        sm100::unpack_f32x2(b2, db[j], db[j + 1]);
      }
    }
    Pack<T> out; out.pack(o);
    st_stream(dX + row * M + col, out.raw);
    x0 = x1; d0 = d1; r0 = r1; m0 = m1;
    if constexpr (!LAYER) { x1 = x2; d1 = d2; r1 = r2; m1 = m2; }
  }
  float4* pw = reinterpret_cast<float4*>(dWp + (size_t)blockIdx.x * M + col);
#pragma unroll
  for (int j = 0; j < VEC; j += 4) pw[j / 4] = make_float4(dw[j], dw[j + 1], dw[j + 2], dw[j + 3]);
  if constexpr (LAYER) {
    float4* pb = reinterpret_cast<float4*>(dBp + (size_t)blockIdx.x * M + col);
#pragma unroll
    for (int j = 0; j < VEC; j += 4) pb[j / 4] = make_float4(db[j], db[j + 1], db[j + 2], db[j + 3]);
  }
}

// backward for any M / alignment: the CTA's partial row is accumulated in global memory
// (the CTA is its only writer).
template <typename T, bool LAYER>
__global__ void __launch_bounds__(256)
norm_bwd_generic_kernel(T* __restrict__ dX, float* __restrict__ dWp, float* __restrict__ dBp,
                        const T* __restrict__ dY, const T* __restrict__ X,
                        const T* __restrict__ W, const float* __restrict__ Mean,
                        const float* __restrict__ Rstd, int64_t M, int64_t N, float offset) {
  __shared__ float red[32];
  const float inv_m = 1.0f / (float)M;
  float* mw = dWp + (size_t)blockIdx.x * M;
  float* mb = LAYER ? dBp + (size_t)blockIdx.x * M : nullptr;
  for (int64_t i = threadIdx.x; i < M; i += 256) { mw[i] = 0.f; if (LAYER) mb[i] = 0.f; }
  for (int64_t row = blockIdx.x; row < N; row += gridDim.x) {
    const T* x = X + row * M; const T* dy = dY + row * M;
    const float rstd = Rstd[row];
    const float mean = LAYER ? Mean[row] : 0.f;
    float s1 = 0.f, s2 = 0.f;
    for (int64_t i = threadIdx.x; i < M; i += 256) {
      const float gi = Elem<T>::to_f(W[i]) + (LAYER ? 0.f : offset);
      const float gd = gi * Elem<T>::to_f(dy[i]);
      s1 += (Elem<T>::to_f(x[i]) - mean) * rstd * gd;
      s2 += gd;
    }
    const float c1 = block_reduce<256>(s1, SumOp(), 0.f, red) * inv_m;
    const float c2 = LAYER ? block_reduce<256>(s2, SumOp(), 0.f, red) * inv_m : 0.f;
    for (int64_t i = threadIdx.x; i < M; i += 256) {
      const float gi = Elem<T>::to_f(W[i]) + (LAYER ? 0.f : offset);
      const float d = Elem<T>::to_f(dy[i]);
      const float xhat = (Elem<T>::to_f(x[i]) - mean) * rstd;
      dX[row * M + i] = Elem<T>::from_f((gi * d - (xhat * c1 + c2)) * rstd);
      mw[i] += d * xhat;
      if (LAYER) mb[i] += d;
    }
  }
}

// second stage: dW[m] = sum over groups of the partial rows.
template <typename T>
__global__ void __launch_bounds__(256)
norm_bwd_reduce_kernel(T* __restrict__ dW, T* __restrict__ dB, const float* __restrict__ dWp,
                       const float* __restrict__ dBp, int64_t M, int n_groups) {
  // 32 columns x 8 group-lanes per CTA
  __shared__ float sw[8][33], sb[8][33];
  const int col = threadIdx.x & 31, gl = threadIdx.x >> 5;
  const int64_t m = (int64_t)blockIdx.x * 32 + col;
  float aw = 0.f, ab = 0.f;
  if (m < M) {
    for (int g = gl; g < n_groups; g += 8) {
      aw += dWp[(size_t)g * M + m];
      if (dBp) ab += dBp[(size_t)g * M + m];
    }
  }
  sw[gl][col] = aw; sb[gl][col] = ab;
  __syncthreads();
  if (gl == 0 && m < M) {
#pragma unroll
    for (int k = 1; k < 8; ++k) { aw += sw[k][col]; ab += sb[k][col]; }
    dW[m] = Elem<T>::from_f(aw);
    if (dBp) dB[m] = Elem<T>::from_f(ab);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
template <typename T, bool LAYER>
static int32_t norm_fwd_launch(void* Y, const void* X, const void* W, const void* Bias, float* Mean,
                               float* Rstd, int64_t M, int64_t N, float eps, float offset,
                               cudaStream_t st) {
  constexpr int VEC = Elem<T>::kVec;
  RowShape shape;
  if (M % VEC == 0 && pick_row_shape(M / VEC, 8, &shape)) {
    TYLO_ROW_DISPATCH(shape, norm_fwd_kernel<T, THREADS, ITERS, LAYER><<<(unsigned)N, THREADS, 0, st>>>(
        (T*)Y, (const T*)X, (const T*)W, (const T*)Bias, Mean, Rstd, (int)M, eps, offset));
  } else {
    norm_fwd_generic_kernel<T, LAYER><<<(unsigned)N, 256, 0, st>>>(
        (T*)Y, (const T*)X, (const T*)W, (const T*)Bias, Mean, Rstd, M, eps, offset);
  }
  return check_launch(LAYER ? "layer_norm_fwd" : "rms_norm_fwd");
}

template <typename T, bool LAYER>
static int32_t norm_bwd_launch(void* dX, void* dW, void* dB, const void* dY, const void* X,
                               const void* W, const float* Mean, const float* Rstd, float* dWp,
                               float* dBp, int n_groups, int64_t M, int64_t N, float offset,
                               cudaStream_t st) {
  constexpr int VEC = Elem<T>::kVec;
  RowShape shape;
  unsigned grid = (unsigned)(n_groups < N ? n_groups : N);
  const int64_t nvec = M % VEC == 0 ? M / VEC : 0;
  if (nvec == 1024 || nvec == 512) {
    // rows of exactly one packet per thread: the streaming form, one CTA per SM (two at 512 threads)
    const unsigned walkers = (unsigned)sm_count() * (nvec == 1024 ? 1u : 2u);
    if (grid > walkers) grid = walkers;
    if (nvec == 1024)
      norm_bwd_stream_kernel<T, 1024, LAYER><<<grid, 1024, 0, st>>>(
          (T*)dX, dWp, dBp, (const T*)dY, (const T*)X, (const T*)W, Mean, Rstd, (int)M, N, offset);
    else
      norm_bwd_stream_kernel<T, 512, LAYER><<<grid, 512, 0, st>>>(
          (T*)dX, dWp, dBp, (const T*)dY, (const T*)X, (const T*)W, Mean, Rstd, (int)M, N, offset);
  } else
  // register-resident shapes only while the per-thread dW/dB accumulators fit without spilling
  if (M % VEC == 0 && M / VEC <= 1024 && pick_row_shape(M / VEC, 4, &shape)) {
#define TYLO_BWD_LAUNCH(THREADS, ITERS)                                                             \
  norm_bwd_kernel<T, THREADS, ITERS, LAYER><<<grid, THREADS, 0, st>>>(                              \
      (T*)dX, dWp, dBp, (const T*)dY, (const T*)X, (const T*)W, Mean, Rstd, (int)M, N, offset)
    if (shape.threads == 32) TYLO_BWD_LAUNCH(32, 2);
    else if (shape.threads == 128) TYLO_BWD_LAUNCH(128, 2);
    else TYLO_BWD_LAUNCH(256, 4);
#undef TYLO_BWD_LAUNCH
  } else {
    norm_bwd_generic_kernel<T, LAYER><<<grid, 256, 0, st>>>(
        (T*)dX, dWp, dBp, (const T*)dY, (const T*)X, (const T*)W, Mean, Rstd, M, N, offset);
  }
  int32_t rc = check_launch(LAYER ? "layer_norm_bwd" : "rms_norm_bwd");
  if (rc) return rc;
  norm_bwd_reduce_kernel<T><<<(unsigned)((M + 31) / 32), 256, 0, st>>>(
      (T*)dW, (T*)dB, dWp, LAYER ? dBp : nullptr, M, (int)grid);
  return check_launch("norm_bwd_reduce");
}

static int32_t check_mn(int64_t M, int64_t N) {
  TYLO_REQUIRE(M > 0 && N > 0, TYLO_ERR_INVALID_ARGUMENT, "extents must be positive (M=%lld, N=%lld)",
               (long long)M, (long long)N);
  TYLO_REQUIRE(N <= 0x7fffffffLL && M <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED,
               "extents above 2^31-1 are not supported (M=%lld, N=%lld)", (long long)M, (long long)N);
  return TYLO_OK;
}

}  // namespace tylo

using namespace tylo;

extern "C" int32_t tylo_b200_rms_norm_fwd(void* Y, const void* X, const void* W, float* Rstd, int64_t M,
                                          int64_t N, float eps, float offset, int32_t dtype,
                                          tylo_stream_t stream) {
  TYLO_REQUIRE(Y && X && W, TYLO_ERR_INVALID_ARGUMENT, "rms_norm_fwd: Y, X and W must be non-null");
  if (int32_t rc = check_mn(M, N)) return rc;
  TYLO_REQUIRE(aligned16(Y) && aligned16(X) && aligned16(W), TYLO_ERR_MISALIGNED,
               "rms_norm_fwd: pointers must be 16-byte aligned");
  TYLO_DISPATCH_DTYPE(dtype, T, return (norm_fwd_launch<T, false>(Y, X, W, nullptr, nullptr, Rstd, M, N, eps,
                                                                  offset, (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_layer_norm_fwd(void* Y, const void* X, const void* W, const void* Bias,
                                            float* Mean, float* Rstd, int64_t M, int64_t N, float eps,
                                            int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(Y && X && W && Bias, TYLO_ERR_INVALID_ARGUMENT,
               "layer_norm_fwd: Y, X, W and B must be non-null");
  if (int32_t rc = check_mn(M, N)) return rc;
  TYLO_REQUIRE(aligned16(Y) && aligned16(X) && aligned16(W) && aligned16(Bias), TYLO_ERR_MISALIGNED,
               "layer_norm_fwd: pointers must be 16-byte aligned");
  TYLO_DISPATCH_DTYPE(dtype, T, return (norm_fwd_launch<T, true>(Y, X, W, Bias, Mean, Rstd, M, N, eps, 0.f,
                                                                 (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_rms_norm_bwd(void* dX, void* dW, const void* dY, const void* X,
                                          const void* W, const float* Rstd, float* dW_partial,
                                          int32_t n_groups, int64_t M, int64_t N, float offset,
                                          int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(dX && dW && dY && X && W && Rstd && dW_partial, TYLO_ERR_INVALID_ARGUMENT,
               "rms_norm_bwd: all pointers must be non-null (Rstd comes from the forward's checkpoints)");
  if (int32_t rc = check_mn(M, N)) return rc;
  TYLO_REQUIRE(n_groups > 0, TYLO_ERR_INVALID_ARGUMENT, "rms_norm_bwd: n_groups must be positive");
  TYLO_REQUIRE(aligned16(dX) && aligned16(dW) && aligned16(dY) && aligned16(X) && aligned16(W) &&
                   aligned16(dW_partial), TYLO_ERR_MISALIGNED,
               "rms_norm_bwd: pointers must be 16-byte aligned");
  TYLO_DISPATCH_DTYPE(dtype, T, return (norm_bwd_launch<T, false>(dX, dW, nullptr, dY, X, W, nullptr, Rstd,
                                                                  dW_partial, nullptr, n_groups, M, N, offset,
                                                                  (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_layer_norm_bwd(void* dX, void* dW, void* dB, const void* dY, const void* X,
                                            const void* W, const float* Mean, const float* Rstd,
                                            float* dW_partial, float* dB_partial, int32_t n_groups,
                                            int64_t M, int64_t N, int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(dX && dW && dB && dY && X && W && Mean && Rstd && dW_partial && dB_partial,
               TYLO_ERR_INVALID_ARGUMENT,
               "layer_norm_bwd: all pointers must be non-null (Mean/Rstd come from the forward's checkpoints)");
  if (int32_t rc = check_mn(M, N)) return rc;
  TYLO_REQUIRE(n_groups > 0, TYLO_ERR_INVALID_ARGUMENT, "layer_norm_bwd: n_groups must be positive");
  TYLO_REQUIRE(aligned16(dX) && aligned16(dW) && aligned16(dB) && aligned16(dY) && aligned16(X) &&
                   aligned16(W) && aligned16(dW_partial) && aligned16(dB_partial), TYLO_ERR_MISALIGNED,
               "layer_norm_bwd: pointers must be 16-byte aligned");
  TYLO_DISPATCH_DTYPE(dtype, T, return (norm_bwd_launch<T, true>(dX, dW, dB, dY, X, W, Mean, Rstd, dW_partial,
                                                                 dB_partial, n_groups, M, N, 0.f,
                                                                 (cudaStream_t)stream)));
  return TYLO_OK;
}
