// Shape- and dtype-generic attention forward / backward in fp32 arithmetic (CUDA cores).
//
// This path serves (a) fp32 storage, where the contract is true-fp32 accuracy (the reference's
// default rounds fp32 operands to TF32, utils.jl:40-44), and (b) every shape or mod combination
// the tcgen05 kernels do not cover (head dims other than 64/128, ragged per-batch lengths, ...).
// It is written for correctness and reasonable speed, not for the roofline: 32x32 tiles staged
// in shared memory as fp32, 256 threads, each owning a 2x2 patch of the score tile and a
// 2 x (D/16) patch of the output tile.
//
// Forward  : one CTA per (32 queries, head, batch), flash-style online softmax.
// Backward : no atomics and no zero-fill.  One kernel owns a 32-key tile of one KV head and sums
//            dK/dV over the query heads of its group in fp32 (attention.jl:192-194 uses
//            storage-dtype atomics); a second kernel owns a 32-query tile and produces dQ
//            (attention.jl:185-187 read-modify-writes dQ in the storage dtype per tile).
#include "attn_params.cuh"

namespace tylo {

constexpr int GT = 32;       // tile edge (queries and keys)
constexpr int GTHREADS = 256;
constexpr int GMAXJ = 16;    // output columns per thread: head dim <= 16 * 16 = 256

template <typename T>
__device__ __forceinline__ void load_tile(float* dst, int ld, const T* __restrict__ src, int row0, int nrows,
                                          int D, int Dpad) {
  for (int idx = threadIdx.x; idx < GT * Dpad; idx += GTHREADS) {
    const int r = idx / Dpad, d = idx % Dpad;
    const int row = row0 + r;
    dst[r * ld + d] = (row < nrows && d < D) ? Elem<T>::to_f(src[(size_t)row * D + d]) : 0.f;
  }
}

__device__ __forceinline__ void dot2x2(const float* A, int lda, const float* Bm, int ldb, int r0, int c0, int D4,
                                       float (&out)[2][2]) {
  float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
  const float4* pa0 = reinterpret_cast<const float4*>(A + r0 * lda);
  const float4* pa1 = reinterpret_cast<const float4*>(A + (r0 + 1) * lda);
  const float4* pb0 = reinterpret_cast<const float4*>(Bm + c0 * ldb);
  const float4* pb1 = reinterpret_cast<const float4*>(Bm + (c0 + 1) * ldb);
  for (int d = 0; d < D4; ++d) {
    const float4 x0 = pa0[d], x1 = pa1[d], y0 = pb0[d], y1 = pb1[d];
    a00 += x0.x * y0.x + x0.y * y0.y + x0.z * y0.z + x0.w * y0.w;
    a01 += x0.x * y1.x + x0.y * y1.y + x0.z * y1.z + x0.w * y1.w;
    a10 += x1.x * y0.x + x1.y * y0.y + x1.z * y0.z + x1.w * y0.w;
    a11 += x1.x * y1.x + x1.y * y1.y + x1.z * y1.z + x1.w * y1.w;
  }
  out[0][0] = a00; out[0][1] = a01; out[1][0] = a10; out[1][1] = a11;
}

__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ int clamp_len(const int32_t* lens, int b, int S) {
  if (!lens) return S;
  const int v = lens[b];
  return v < 0 ? 0 : (v > S ? S : v);
}
// attention.jl:25-26 skips whole 64-row query blocks that start at or beyond q_lengths[b].
__device__ __forceinline__ int q_row_limit(const AttnParams& p, int b) {
  if (!p.q_lengths) return p.Sq;
  const int ql = clamp_len(p.q_lengths, b, p.Sq);
  const int lim = ((ql + 63) / 64) * 64;
  return lim < p.Sq ? lim : p.Sq;
}
__device__ __forceinline__ float lse2_of(const AttnParams& p, float M, float L) {
  if (!(L > 0.f)) return -INFINITY;
  return (p.natural_stats ? M * kLog2e : M) + log2f(L);
}

// -------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(GTHREADS)
attn_fwd_generic_kernel(T* __restrict__ O, const T* __restrict__ Q, const T* __restrict__ K,
                        const T* __restrict__ V, float* __restrict__ Mout, float* __restrict__ Lout,
                        AttnParams p) {
  extern __shared__ __align__(16) float gsm[];
  const int Dk4 = (p.Dk + 3) & ~3, ldk = Dk4 + 4;
  float* sQ = gsm;
  float* sK = sQ + GT * ldk;
  float* sV = sK + GT * ldk;
  float* sP = sV + GT * p.Dv;   // [GT][GT+1]

  const int nqt = (p.Sq + GT - 1) / GT;
  const int qt = blockIdx.x % nqt, hb = blockIdx.x / nqt;
  const int b = hb / p.H, h = hb % p.H, hk = h / p.G;
  const int q0 = qt * GT;
  if (q0 >= q_row_limit(p, b)) return;
  const int k_len = clamp_len(p.k_lengths, b, p.Sk);

  const T* Qg = Q + ((size_t)(b * p.H + h) * p.Sq) * p.Dk;
  const T* Kg = K + ((size_t)(b * p.Hkv + hk) * p.Sk) * p.Dk;
  const T* Vg = V + ((size_t)(b * p.Hkv + hk) * p.Sk) * p.Dv;
  load_tile(sQ, ldk, Qg, q0, p.Sq, p.Dk, Dk4);

  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int r0 = 2 * ty, c0 = 2 * tx;
  const float slope = (p.score_flags & TYLO_SCORE_ALIBI) ? p.slopes[h] : 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[2][GMAXJ];
#pragma unroll
  for (int j = 0; j < GMAXJ; ++j) { o[0][j] = 0.f; o[1][j] = 0.f; }

  // one 32-key tile; use_mask = false skips the mask mod (a block the host marked fully unmasked)
  auto key_tile = [&](const int kv0, const bool use_mask) {
    __syncthreads();
    load_tile(sK, ldk, Kg, kv0, p.Sk, p.Dk, Dk4);
    load_tile(sV, p.Dv, Vg, kv0, p.Sk, p.Dv, p.Dv);
    __syncthreads();
    float s[2][2];
    dot2x2(sQ, ldk, sK, ldk, r0, c0, Dk4 / 4, s);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = q0 + r0 + i, qpos = row + p.input_pos;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kv = kv0 + c0 + j;
        const bool ok = row < p.Sq && kv < k_len && (!use_mask || mask_keep(p, b, qpos, kv));
        s[i][j] = ok ? score_apply(p, s[i][j] * p.scale, score_additive(p, slope, b, h, row, qpos, kv)) * kLog2e : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
      mx = half_warp_max(mx);
      const float mn = fmaxf(m[i], mx);
      const float alpha = (mn == -INFINITY) ? 1.f : exp2f(m[i] - mn);
      float ps = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float pv = (s[i][j] == -INFINITY) ? 0.f : exp2f(s[i][j] - mn);
        sP[(r0 + i) * (GT + 1) + c0 + j] = pv;
        ps += pv;
      }
      ps = half_warp_sum(ps);
      l[i] = l[i] * alpha + ps;
      m[i] = mn;
#pragma unroll
      for (int j = 0; j < GMAXJ; ++j) o[i][j] *= alpha;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < GMAXJ; ++j) {
      const int c = tx + 16 * j;
      if (c < p.Dv) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
        for (int n = 0; n < GT; ++n) {
          const float v = sV[n * p.Dv + c];
          a0 += sP[r0 * (GT + 1) + n] * v;
          a1 += sP[(r0 + 1) * (GT + 1) + n] * v;
        }
        o[0][j] += a0; o[1][j] += a1;
      }
    }
  };
  if (p.bm_count) {
    // walk the host-built block list of this query block (flex.jl:107-182); tile edges are multiples of GT
    const int qb = q0 / p.bm_tm;
    const int nb = min(p.bm_count[qb], p.bm_stride);
    for (int t = 0; t < nb; ++t) {
      const int j = p.bm_idx[(size_t)qb * p.bm_stride + t];
      const bool full = p.bm_full[(size_t)qb * p.bm_stride + t] != 0;
      if (j < 0) continue;
      const int kend = min((j + 1) * p.bm_tn, p.Sk);
      for (int kv0 = j * p.bm_tn; kv0 < kend; kv0 += GT) key_tile(kv0, !full);
    }
  } else {
    int lo, hi;
    kv_range(p, q0 + p.input_pos, min(q0 + GT, p.Sq) - 1 + p.input_pos, k_len, &lo, &hi);
    for (int kv0 = (lo / GT) * GT; kv0 < hi; kv0 += GT) key_tile(kv0, true);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = q0 + r0 + i;
    if (row >= p.Sq) continue;
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    T* og = O + ((size_t)(b * p.H + h) * p.Sq + row) * p.Dv;
#pragma unroll
    for (int j = 0; j < GMAXJ; ++j) {
      const int c = tx + 16 * j;
      if (c < p.Dv) og[c] = Elem<T>::from_f(o[i][j] * inv);
    }
    if (tx == 0) {
      const size_t si = (size_t)(b * p.H + h) * p.Sq + row;
      if (Mout) Mout[si] = p.natural_stats ? m[i] * kLn2 : m[i];
      if (Lout) Lout[si] = l[i];
    }
  }
}

// Delta[row] = sum_d dO * O  (the reference's preprocess, attention.jl:90-117, computes the same
// quantity on dO / L; here dO stays unscaled and P is normalised through the log-sum-exp).
template <typename T>
__global__ void __launch_bounds__(256)
attn_bwd_delta_kernel(float* __restrict__ Delta, const T* __restrict__ O, const T* __restrict__ dO,
                      long long rows, int Dv) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int d = lane; d < Dv; d += 32)
    s += Elem<T>::to_f(O[(size_t)row * Dv + d]) * Elem<T>::to_f(dO[(size_t)row * Dv + d]);
  s = warp_reduce(s, SumOp());
  if (lane == 0) Delta[row] = s;
}

// Host-built block list (mods.jl:436-476) seen from one 32x32 tile: 0 = its (query block, key block) is
// not listed, 1 = listed, 2 = listed and marked fully unmasked.  Block ids of one query block are distinct.
__device__ __forceinline__ int bm_state(const AttnParams& p, int q0, int kv0) {
  const int qb = q0 / p.bm_tm, kb = kv0 / p.bm_tn;
  const int nb = min(p.bm_count[qb], p.bm_stride);
  int st = 0;
  for (int t = 0; t < nb; ++t)
    if (p.bm_idx[(size_t)qb * p.bm_stride + t] == kb) st = max(st, p.bm_full[(size_t)qb * p.bm_stride + t] != 0 ? 2 : 1);
  return st;
}

// Shared by both backward kernels: for the thread's 2x2 patch compute p and the scaled
// pre-mod score gradient.  Returns the ALiBi slope-gradient contribution of the patch.
struct BwdPatch { float p[2][2], ds0[2][2]; };

template <bool PARAM_GRADS>
__device__ __forceinline__ float bwd_patch(const AttnParams& p, int b, int h, float slope, const float* sQ,
                                           const float* sK, const float* sdO, const float* sV, int ldk,
                                           int ldv, int Dk4, int Dv4, int q0, int kv0, int r0, int c0,
                                           int q_lim, int k_len, const float* sLse, const float* sDelta,
                                           BwdPatch& out, const bool use_mask) {
  float s[2][2], dp[2][2];
  dot2x2(sQ, ldk, sK, ldk, r0, c0, Dk4 / 4, s);
  dot2x2(sdO, ldv, sV, ldv, r0, c0, Dv4 / 4, dp);
  float slope_acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = q0 + r0 + i, qpos = row + p.input_pos;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int kv = kv0 + c0 + j;
      const bool ok = row < q_lim && kv < k_len && (!use_mask || mask_keep(p, b, qpos, kv));
      float pv = 0.f, g0 = 0.f;
      if (ok) {
        const float s0 = s[i][j] * p.scale;
        const float add = score_additive(p, slope, b, h, row, qpos, kv);
        const float t = score_apply(p, s0, add) * kLog2e;
        const float lse = sLse[r0 + i];
        pv = (lse == -INFINITY) ? 0.f : exp2f(t - lse);
        const float ds = pv * (dp[i][j] - sDelta[r0 + i]);
        float at_add;
        g0 = score_vjp(p, s0, add, ds, &at_add);
        slope_acc += at_add * (float)(qpos - kv);
        // broadcast heads / batch entries share a table entry: accumulate atomically (mods.jl:305-313)
        if (PARAM_GRADS && p.d_bias && (p.score_flags & TYLO_SCORE_BIAS)) atomicAdd(p.d_bias + bias_index(p, b, h, row, kv), at_add);
      }
      out.p[i][j] = pv;
      out.ds0[i][j] = g0 * p.scale;
    }
  }
  return slope_acc;
}

template <typename T>
__global__ void __launch_bounds__(GTHREADS)
attn_bwd_dkdv_generic_kernel(T* __restrict__ dK, T* __restrict__ dV, const T* __restrict__ Q,
                             const T* __restrict__ K, const T* __restrict__ V, const T* __restrict__ dO,
                             const float* __restrict__ Mst, const float* __restrict__ Lst,
                             const float* __restrict__ Delta, AttnParams p) {
  extern __shared__ __align__(16) float gsm[];
  const int Dk4 = (p.Dk + 3) & ~3, ldk = Dk4 + 4;
  const int Dv4 = (p.Dv + 3) & ~3, ldv = Dv4 + 4;
  float* sQ = gsm;
  float* sK = sQ + GT * ldk;
  float* sdO = sK + GT * ldk;
  float* sV = sdO + GT * ldv;
  float* sP = sV + GT * ldv;          // [GT][GT+1]
  float* sdS = sP + GT * (GT + 1);    // [GT][GT+1]
  float* sLse = sdS + GT * (GT + 1);  // [GT]
  float* sDelta = sLse + GT;          // [GT]

  const int nkt = (p.Sk + GT - 1) / GT;
  const int kt = blockIdx.x % nkt, hkb = blockIdx.x / nkt;
  const int b = hkb / p.Hkv, hk = hkb % p.Hkv;
  const int kv0 = kt * GT;
  const int k_len = clamp_len(p.k_lengths, b, p.Sk);
  const int q_lim = q_row_limit(p, b);

  const T* Kg = K + ((size_t)(b * p.Hkv + hk) * p.Sk) * p.Dk;
  const T* Vg = V + ((size_t)(b * p.Hkv + hk) * p.Sk) * p.Dv;
  load_tile(sK, ldk, Kg, kv0, p.Sk, p.Dk, Dk4);
  load_tile(sV, ldv, Vg, kv0, p.Sk, p.Dv, Dv4);

  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int r0 = 2 * ty, c0 = 2 * tx;
  float dk[2][GMAXJ], dv[2][GMAXJ];
#pragma unroll
  for (int j = 0; j < GMAXJ; ++j) { dk[0][j] = dk[1][j] = dv[0][j] = dv[1][j] = 0.f; }

  int qlo, qhi;
  q_range(p, kv0, min(kv0 + GT, p.Sk) - 1, q_lim, &qlo, &qhi);
  if (kv0 >= k_len) qhi = qlo;  // keys beyond the valid length receive zero gradient
  for (int g = 0; g < p.G; ++g) {
    const int h = hk * p.G + g;
    const float slope = (p.score_flags & TYLO_SCORE_ALIBI) ? p.slopes[h] : 0.f;
    const T* Qg = Q + ((size_t)(b * p.H + h) * p.Sq) * p.Dk;
    const T* dOg = dO + ((size_t)(b * p.H + h) * p.Sq) * p.Dv;
    const size_t sbase = (size_t)(b * p.H + h) * p.Sq;
    for (int q0 = (qlo / GT) * GT; q0 < qhi; q0 += GT) {
      const int listed = p.bm_count ? bm_state(p, q0, kv0) : 1;   // uniform over the CTA
      if (listed == 0) continue;
      __syncthreads();
      load_tile(sQ, ldk, Qg, q0, p.Sq, p.Dk, Dk4);
      load_tile(sdO, ldv, dOg, q0, p.Sq, p.Dv, Dv4);
      if (threadIdx.x < GT) {
        const int row = q0 + threadIdx.x;
        sLse[threadIdx.x] = row < q_lim ? lse2_of(p, Mst[sbase + row], Lst[sbase + row]) : -INFINITY;
        sDelta[threadIdx.x] = row < q_lim ? Delta[sbase + row] : 0.f;
      }
      __syncthreads();
      BwdPatch bp;
      bwd_patch<false>(p, b, h, slope, sQ, sK, sdO, sV, ldk, ldv, Dk4, Dv4, q0, kv0, r0, c0, q_lim, k_len, sLse, sDelta, bp,
                       listed != 2);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          sP[(r0 + i) * (GT + 1) + c0 + j] = bp.p[i][j];
          sdS[(r0 + i) * (GT + 1) + c0 + j] = bp.ds0[i][j];
        }
      __syncthreads();
      // this thread owns key rows r0, r0+1 of the tile and columns tx + 16 j
#pragma unroll
      for (int j = 0; j < GMAXJ; ++j) {
        const int c = tx + 16 * j;
        if (c < p.Dv) {
          float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
          for (int mrow = 0; mrow < GT; ++mrow) {
            const float d = sdO[mrow * ldv + c];
            a0 += sP[mrow * (GT + 1) + r0] * d;
            a1 += sP[mrow * (GT + 1) + r0 + 1] * d;
          }
          dv[0][j] += a0; dv[1][j] += a1;
        }
        if (c < p.Dk) {
          float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
          for (int mrow = 0; mrow < GT; ++mrow) {
            const float qv = sQ[mrow * ldk + c];
            a0 += sdS[mrow * (GT + 1) + r0] * qv;
            a1 += sdS[mrow * (GT + 1) + r0 + 1] * qv;
          }
          dk[0][j] += a0; dk[1][j] += a1;
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int kv = kv0 + r0 + i;
    if (kv >= p.Sk) continue;
    T* dkg = dK + ((size_t)(b * p.Hkv + hk) * p.Sk + kv) * p.Dk;
    T* dvg = dV + ((size_t)(b * p.Hkv + hk) * p.Sk + kv) * p.Dv;
#pragma unroll
    for (int j = 0; j < GMAXJ; ++j) {
      const int c = tx + 16 * j;
      if (c < p.Dk) dkg[c] = Elem<T>::from_f(dk[i][j]);
      if (c < p.Dv) dvg[c] = Elem<T>::from_f(dv[i][j]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(GTHREADS)
attn_bwd_dq_generic_kernel(T* __restrict__ dQ, const T* __restrict__ Q, const T* __restrict__ K,
                           const T* __restrict__ V, const T* __restrict__ dO, const float* __restrict__ Mst,
                           const float* __restrict__ Lst, const float* __restrict__ Delta, AttnParams p) {
  extern __shared__ __align__(16) float gsm[];
  __shared__ float red[32];
  const int Dk4 = (p.Dk + 3) & ~3, ldk = Dk4 + 4;
  const int Dv4 = (p.Dv + 3) & ~3, ldv = Dv4 + 4;
  float* sQ = gsm;
  float* sK = sQ + GT * ldk;
  float* sdO = sK + GT * ldk;
  float* sV = sdO + GT * ldv;
  float* sdS = sV + GT * ldv;          // [GT][GT+1]
  float* sLse = sdS + GT * (GT + 1);
  float* sDelta = sLse + GT;

  const int nqt = (p.Sq + GT - 1) / GT;
  const int qt = blockIdx.x % nqt, hb = blockIdx.x / nqt;
  const int b = hb / p.H, h = hb % p.H, hk = h / p.G;
  const int q0 = qt * GT;
  const int k_len = clamp_len(p.k_lengths, b, p.Sk);
  const int q_lim = q_row_limit(p, b);
  const float slope = (p.score_flags & TYLO_SCORE_ALIBI) ? p.slopes[h] : 0.f;

  const T* Qg = Q + ((size_t)(b * p.H + h) * p.Sq) * p.Dk;
  const T* dOg = dO + ((size_t)(b * p.H + h) * p.Sq) * p.Dv;
  const T* Kg = K + ((size_t)(b * p.Hkv + hk) * p.Sk) * p.Dk;
  const T* Vg = V + ((size_t)(b * p.Hkv + hk) * p.Sk) * p.Dv;
  const size_t sbase = (size_t)(b * p.H + h) * p.Sq;
  load_tile(sQ, ldk, Qg, q0, p.Sq, p.Dk, Dk4);
  load_tile(sdO, ldv, dOg, q0, p.Sq, p.Dv, Dv4);
  if (threadIdx.x < GT) {
    const int row = q0 + threadIdx.x;
    sLse[threadIdx.x] = row < q_lim ? lse2_of(p, Mst[sbase + row], Lst[sbase + row]) : -INFINITY;
    sDelta[threadIdx.x] = row < q_lim ? Delta[sbase + row] : 0.f;
  }

  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const int r0 = 2 * ty, c0 = 2 * tx;
  float dq[2][GMAXJ];
#pragma unroll
  for (int j = 0; j < GMAXJ; ++j) { dq[0][j] = dq[1][j] = 0.f; }
  float slope_acc = 0.f;

  int lo, hi;
  kv_range(p, q0 + p.input_pos, min(q0 + GT, p.Sq) - 1 + p.input_pos, k_len, &lo, &hi);
  if (q0 >= q_lim) hi = lo;
  for (int kv0 = (lo / GT) * GT; kv0 < hi; kv0 += GT) {
    const int listed = p.bm_count ? bm_state(p, q0, kv0) : 1;   // uniform over the CTA
    if (listed == 0) continue;
    __syncthreads();
    load_tile(sK, ldk, Kg, kv0, p.Sk, p.Dk, Dk4);
    load_tile(sV, ldv, Vg, kv0, p.Sk, p.Dv, Dv4);
    __syncthreads();
    BwdPatch bp;
    slope_acc += bwd_patch<true>(p, b, h, slope, sQ, sK, sdO, sV, ldk, ldv, Dk4, Dv4, q0, kv0, r0, c0, q_lim, k_len,
                           sLse, sDelta, bp, listed != 2);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) sdS[(r0 + i) * (GT + 1) + c0 + j] = bp.ds0[i][j];
    __syncthreads();
#pragma unroll
    for (int j = 0; j < GMAXJ; ++j) {
      const int c = tx + 16 * j;
      if (c < p.Dk) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
        for (int n = 0; n < GT; ++n) {
          const float kvv = sK[n * ldk + c];
          a0 += sdS[r0 * (GT + 1) + n] * kvv;
          a1 += sdS[(r0 + 1) * (GT + 1) + n] * kvv;
        }
        dq[0][j] += a0; dq[1][j] += a1;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = q0 + r0 + i;
    if (row >= p.Sq) continue;
    T* dqg = dQ + ((size_t)(b * p.H + h) * p.Sq + row) * p.Dk;
#pragma unroll
    for (int j = 0; j < GMAXJ; ++j) {
      const int c = tx + 16 * j;
      if (c < p.Dk) dqg[c] = Elem<T>::from_f(dq[i][j]);
    }
  }
  if (p.d_slopes && (p.score_flags & TYLO_SCORE_ALIBI)) {
    __syncthreads();
    // ds0 carries the qk scale; the slope gradient is taken on the unscaled score gradient
    slope_acc = block_reduce<GTHREADS>(slope_acc, SumOp(), 0.f, red);
    if (threadIdx.x == 0) atomicAdd(p.d_slopes + h, slope_acc);
  }
}

// -------------------------------------------------------------------------------------------------
template <typename T>
int32_t attn_fwd_generic(void* O, const void* Q, const void* K, const void* V, float* M, float* L,
                         const AttnParams& p, cudaStream_t st) {
  TYLO_REQUIRE(p.Dk <= 256 && p.Dv <= 256, TYLO_ERR_UNSUPPORTED,
               "attention: head dims above 256 are not supported (Dk=%d, Dv=%d)", p.Dk, p.Dv);
  const int Dk4 = (p.Dk + 3) & ~3;
  const size_t smem = sizeof(float) * (2 * GT * (Dk4 + 4) + GT * p.Dv + GT * (GT + 1));
  auto kern = attn_fwd_generic_kernel<T>;
  TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long long grid = (long long)((p.Sq + GT - 1) / GT) * p.H * p.B;
  TYLO_REQUIRE(grid <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED, "attention: problem too large for one launch");
  kern<<<(unsigned)grid, GTHREADS, smem, st>>>((T*)O, (const T*)Q, (const T*)K, (const T*)V, M, L, p);
  return check_launch("attn_fwd_generic");
}

template <typename T>
int32_t attn_bwd_generic(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V,
                         const void* O, const void* dO, const float* M, const float* L, float* Delta,
                         const AttnParams& p, cudaStream_t st) {
  TYLO_REQUIRE(p.Dk <= 256 && p.Dv <= 256, TYLO_ERR_UNSUPPORTED,
               "attention backward: head dims above 256 are not supported (Dk=%d, Dv=%d)", p.Dk, p.Dv);
  const long long rows = (long long)p.Sq * p.H * p.B;
  attn_bwd_delta_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(Delta, (const T*)O, (const T*)dO, rows, p.Dv);
  if (int32_t rc = check_launch("attn_bwd_delta")) return rc;
  const int Dk4 = (p.Dk + 3) & ~3, Dv4 = (p.Dv + 3) & ~3;
  const size_t smem = sizeof(float) * (2 * GT * (Dk4 + 4) + 2 * GT * (Dv4 + 4) + 2 * GT * (GT + 1) + 2 * GT);
  {
    auto kern = attn_bwd_dkdv_generic_kernel<T>;
    TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long grid = (long long)((p.Sk + GT - 1) / GT) * p.Hkv * p.B;
    TYLO_REQUIRE(grid <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED, "attention backward: problem too large");
    kern<<<(unsigned)grid, GTHREADS, smem, st>>>((T*)dK, (T*)dV, (const T*)Q, (const T*)K, (const T*)V,
                                                 (const T*)dO, M, L, Delta, p);
    if (int32_t rc = check_launch("attn_bwd_dkdv_generic")) return rc;
  }
  {
    auto kern = attn_bwd_dq_generic_kernel<T>;
    TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long grid = (long long)((p.Sq + GT - 1) / GT) * p.H * p.B;
    TYLO_REQUIRE(grid <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED, "attention backward: problem too large");
    kern<<<(unsigned)grid, GTHREADS, smem, st>>>((T*)dQ, (const T*)Q, (const T*)K, (const T*)V, (const T*)dO, M,
                                                 L, Delta, p);
    if (int32_t rc = check_launch("attn_bwd_dq_generic")) return rc;
  }
  return TYLO_OK;
}

#define TYLO_INSTANTIATE(T)                                                                                   \
  template int32_t attn_fwd_generic<T>(void*, const void*, const void*, const void*, float*, float*,          \
                                       const AttnParams&, cudaStream_t);                                      \
  template int32_t attn_bwd_generic<T>(void*, void*, void*, const void*, const void*, const void*,            \
                                       const void*, const void*, const float*, const float*, float*,          \
                                       const AttnParams&, cudaStream_t);
TYLO_INSTANTIATE(float)
TYLO_INSTANTIATE(__nv_bfloat16)
TYLO_INSTANTIATE(__half)

}  // namespace tylo
