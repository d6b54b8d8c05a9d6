// Flash-attention backward for sm_100a on tcgen05 / TMEM / TMA, as two launches of one template.
//
//   mode DKDV  one CTA owns 128 keys of one KV head and streams the query tiles that can see them
//              (all G query heads of the group in turn).  Everything is computed TRANSPOSED so that
//              TMEM lanes are keys:
//                 T1 = K Q^T  (= S^T)        T2 = V dO^T (= dP^T)        both operands in shared memory
//                 U1 = P^T,  U2 = dS^T       written back over T1 / T2 as 16-bit
//                 dV += U1 dO                dK += U2 Q                  A from tensor memory (full rate)
//              dK and dV stay in TMEM over the whole group: the GQA sum is fp32 and needs no atomics.
//   mode DQ    one CTA owns 128 queries of one head and streams the key tiles: T1 = Q K^T, T2 = dO V^T,
//              U2 = dS, dQ += U2 K.
//
// Recomputing S and dP in both modes costs 7 tile MMAs per (q,kv) tile pair instead of 5, and in
// exchange there is no fp32 dQ workspace, no atomic traffic, no zero-fill, and results are
// bit-repeatable (the reference read-modify-writes dQ in the storage type per tile and uses
// storage-type atomics for GQA: attention.jl:185-194).
//
// Roles per CTA (384 threads): warp 0 = producer (TMA tiles; in DKDV also the per-query statistics
// of each streamed tile), warp 1 = MMA issuer and TMEM owner, warps 4-7 and 8-11 = two compute
// warpgroups that split the 128 columns of T1/T2 in halves; thread r of each owns TMEM lane r.
// P uses the forward's saved statistics through lse2 = log2-domain log-sum-exp, so the element work
// has no reductions: p = exp2(t - lse2), ds = p (dp - Delta).
//
// U (16-bit, two values per column) of column half w overwrites T columns [64w, 64w+32).
// TMEM columns: [0,128) T1/U1, [128,256) T2/U2, [256,256+D) acc1 (dV), [384,384+D) acc2 (dK or dQ).
// No multicast, no clusters; every wait is bounded (see sm100_ptx.cuh).
#include <cuda.h>
#include <cudaTypedefs.h>

#include "attn_dispatch.cuh"
#include "sm100_ptx.cuh"

namespace tylo {
using namespace sm100;

__device__ int g_attn_bwd_status = 0;

namespace bwd {

constexpr int BT = 128;            // tile edge (queries and keys)
constexpr int kThreads = 384;
constexpr int kStages = 2;
enum Mode { DKDV = 0, DQ = 1 };

template <int D> struct Smem {
  static constexpr int kTile = BT * D * 2;
  static constexpr int kX = 0;                               // two stationary tiles
  static constexpr int kY = 2 * kTile;                       // ring of (Y1, Y2) pairs
  static constexpr int kStats = kY + kStages * 2 * kTile;    // per stage: lse2[128], delta[128], doc[128]
  static constexpr int kStatStage = 3 * BT * 4 + 16;         // + smallest / largest document id of the tile
  static constexpr int kBars = kStats + kStages * kStatStage;
  static constexpr int X_FULL = 0, Y_FULL = 1, Y_EMPTY = Y_FULL + kStages, STAT_FULL = Y_EMPTY + kStages,
                       T1_FULL = STAT_FULL + kStages, T2_FULL = T1_FULL + 1, U1_FULL = T2_FULL + 1, U2_FULL = U1_FULL + 1, DONE = U2_FULL + 1,
                       kNumBars = DONE + 1;
  static constexpr int kMisc = kBars + 8 * kNumBars;
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

template <typename T> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr int v = 1; };
template <> struct Fmt<__half> { static constexpr int v = 0; };

template <typename T> __device__ __forceinline__ uint32_t pack16(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack16<__nv_bfloat16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack16<__half>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// tanh(x): odd polynomial on the FMA pipe for small |x|, hardware approximation otherwise
__device__ __forceinline__ float tanh_fast(float x) {
  const float x2 = x * x;
  float t;
  if (x2 < 0.16f) t = x * fmaf(x2, fmaf(x2, fmaf(x2, -0.05396825f, 0.13333334f), -0.33333334f), 1.f);
  else asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
__device__ __forceinline__ void tmem_st32x(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 16-byte shared-memory load into four registers (explicit shared-space address: no generic
// addressing, no array the compiler would have to keep in local memory)
__device__ __forceinline__ void lds128(uint32_t saddr, float& a, float& b, float& c, float& d) {
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(a), "=f"(b), "=f"(c), "=f"(d) : "r"(saddr));
}
__device__ __forceinline__ void lds128i(uint32_t saddr, int& a, int& b, int& c, int& d) {
  asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(saddr));
}
__device__ __forceinline__ void tmem_st16x(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// p and the scaled pre-mod score gradient for one element.
//   s   : raw dot product q.k          dp : dO.v          lse2 / delta : statistics of the query
// Returns p; ds0 (already multiplied by the qk scale) through the reference.
//   nlse, ndelta : the statistics NEGATED (so that they enter as addends of fused multiply-adds)
//   keep : the pair survives the mask (only read when PARTIAL)     q_minus_kv : position difference (ALiBi)
//   ds_add : gradient at the additive mods' place in the chain (mods.jl:296-303): times (q - kv) it sums
//            to the ALiBi slope gradient; a soft cap applied after the additive mod is already in it
template <bool MODDED, bool PARTIAL>
//   bias : BiasScore's table entry for the pair (mods.jl:219-237), added where ALiBi adds
__device__ __forceinline__ float element(const AttnParams& p, float c, float slope, float inv_cap, float s, float dp,
                                         float nlse, float ndelta, int q_minus_kv, bool keep, float bias, float& ds0,
                                         float& ds_add) {
  float pv, f_inner = p.scale, f_outer = 1.f;
  if (MODDED) {
    float s0 = s * p.scale, sm = s0;
    const bool alibi = p.score_flags & TYLO_SCORE_ALIBI, cap = p.score_flags & TYLO_SCORE_SOFTCAP;
    const bool cap_first = p.score_flags & TYLO_SCORE_SOFTCAP_FIRST;
    if (cap && cap_first) { const float t = tanh_fast(sm * inv_cap); sm = p.cap * t; f_inner *= (1.f - t * t); }
    if (alibi) sm = fmaf(slope, (float)q_minus_kv, sm);
    if (p.score_flags & TYLO_SCORE_BIAS) sm += bias;
    if (cap && !cap_first) { const float t = tanh_fast(sm * inv_cap); sm = p.cap * t; f_outer = (1.f - t * t); }
    pv = ex2(fmaf(sm, kLog2e, nlse));
  } else {
    pv = ex2(fmaf(s, c, nlse));
  }
  if (PARTIAL) {
    if (!keep) pv = 0.f;
  }
  ds_add = pv * (dp + ndelta) * f_outer;
  ds0 = ds_add * f_inner;
  return pv;
}

// The streamed positions a row of the owned tile can pair with under every mask term except the
// document comparison: one interval [lo, hi] of row indices of the streamed tensor (queries for a key
// row in DKDV mode, keys for a query row in DQ mode); mods.jl:101-167 reduced to bounds.
// k_len: keys of this batch entry that exist; q_lim: query rows below it take part (ragged batches).
//   m, window, prefix_len : the conjunction's terms (the mask itself, or one OR-ed clause of it, mods.jl:164-167)
__device__ __forceinline__ bool row_interval(const AttnParams& p, uint32_t m, int window, int prefix_len, bool keys_own,
                                             int own_row, int k_len, int q_lim, int* lo_out, int* hi_out) {
  int lo = 0, hi;
  bool any;
  if (keys_own) {                      // own row = key kv, streamed = query rows q (position q + input_pos)
    const int kv = own_row;
    hi = q_lim - 1;
    any = kv < k_len;
    if (m & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) lo = max(lo, kv - p.input_pos);
    if (m & TYLO_MASK_SLIDING) hi = min(hi, kv + window - p.input_pos);
    if ((m & TYLO_MASK_PREFIX) && kv >= prefix_len) any = false;
    if ((m & TYLO_MASK_PREFIX_LM) && kv >= prefix_len) lo = max(lo, kv - p.input_pos);
  } else {                             // own row = query, streamed = keys
    const int qpos = own_row + p.input_pos;
    hi = k_len - 1;
    any = own_row < q_lim;
    if (m & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) hi = min(hi, qpos);
    if (m & TYLO_MASK_SLIDING) lo = max(lo, qpos - window);
    if (m & TYLO_MASK_PREFIX) hi = min(hi, prefix_len - 1);
    if (m & TYLO_MASK_PREFIX_LM) hi = min(hi, max(qpos, prefix_len - 1));
  }
  *lo_out = lo; *hi_out = hi;
  return any && hi >= lo;
}

// ORS: the instantiation that also evaluates OR-ed mask clauses; the common one carries none of that code (with
// it, the register allocation of the plain element passes changed enough to cost them 3-4 %).
template <typename T, int D, int MODE, bool ORS>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                      T* __restrict__ out1, T* __restrict__ out2, const float* __restrict__ lse2g,
                      const float* __restrict__ deltag, const AttnParams p) {
  using SM = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_addr(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMisc + 4);
  auto bar = [&](int i) { return sbase + SM::kBars + 8 * i; };
  auto stat = [&](int s, int which) { return reinterpret_cast<float*>(smem + SM::kStats + s * SM::kStatStage + which * BT * 4); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // dK/dV kernel: once its last CTAs are resident, the dQ kernel behind it may start filling idle SMs
  if (MODE == DKDV) asm volatile("griddepcontrol.launch_dependents;");

  // ---- what this CTA owns and which tiles it streams
  int b, h0, hk, own0;       // own0: first row (key or query) of the owned tile
  int it_lo, it_n, n_iter;   // streamed tile range [it_lo, it_lo + it_n) per head; n_iter over the group
  // Ragged batches (attention.jl:25-26,60): keys at or beyond k_lengths[b] do not exist; 64-row query
  // blocks starting at or beyond q_lengths[b] were skipped by the forward and take no part here.
  int k_len = p.Sk, q_lim = p.Sq;
  auto batch_lengths = [&](int bb) {
    if (p.k_lengths) { const int v = p.k_lengths[bb]; k_len = v < 0 ? 0 : (v > p.Sk ? p.Sk : v); }
    if (p.q_lengths) {
      const int v = p.q_lengths[bb];
      const int ql = v < 0 ? 0 : (v > p.Sq ? p.Sq : v);
      q_lim = min(p.Sq, ((ql + 63) / 64) * 64);
    }
  };
  if (MODE == DKDV) {
    const int nkt = (p.Sk + BT - 1) / BT;
    const int nhkb = p.Hkv * p.B;
    const int kt = blockIdx.x / nhkb, hkb = blockIdx.x % nhkb;   // key tile slowest: under a causal mask the
    (void)nkt;                                                    // low tiles carry the most work and start first
    b = hkb / p.Hkv; hk = hkb % p.Hkv; h0 = hk * p.G; own0 = kt * BT;
    batch_lengths(b);
    int lo = 0, hi = 0;
    if (own0 < k_len) q_range(p, own0, min(own0 + BT, k_len) - 1, q_lim, &lo, &hi);
    it_lo = lo / BT; it_n = hi > lo ? (hi - 1) / BT - it_lo + 1 : 0;
    n_iter = it_n * p.G;
  } else {
    const int nqt = (p.Sq + BT - 1) / BT;
    const int qt = nqt - 1 - (int)(blockIdx.x % nqt), hb = blockIdx.x / nqt;
    b = hb / p.H; h0 = hb % p.H; hk = h0 / p.G; own0 = qt * BT;
    batch_lengths(b);
    int lo = 0, hi = 0;
    if (own0 < q_lim) kv_range(p, own0 + p.input_pos, min(own0 + BT, q_lim) - 1 + p.input_pos, k_len, &lo, &hi);
    it_lo = lo / BT; it_n = hi > lo ? (hi - 1) / BT - it_lo + 1 : 0;
    n_iter = it_n;
  }

  if (threadIdx.x == 0) {
    mbar_init(bar(SM::X_FULL), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(SM::Y_FULL + s), 1); mbar_init(bar(SM::Y_EMPTY + s), 1); mbar_init(bar(SM::STAT_FULL + s), 32);
    }
    mbar_init(bar(SM::T1_FULL), 1); mbar_init(bar(SM::T2_FULL), 1);
    mbar_init(bar(SM::U1_FULL), 256); mbar_init(bar(SM::U2_FULL), 256);
    mbar_init(bar(SM::DONE), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_addr(tmem_slot), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Register split 4 x 32 x 72 + 8 x 32 x 216 of the launch-time pool: with 56 registers the producer
  // and MMA-issuing threads spill on the hand-off path (measured +2.7 % for 72 / 216; 88 / 208 moves the
  // spills into the element warps and gains nothing).
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 0 && n_iter > 0) {
      // ------------------------------------------------------------------ producer (whole warp)
      if (lane == 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmdO);
        mbar_expect_tx(bar(SM::X_FULL), 2 * SM::kTile);
#pragma unroll
        for (int cc = 0; cc < D / 64; ++cc) {
          if (MODE == DKDV) {
            tma_load_3d(sbase + SM::kX + cc * (BT * 128), &tmK, bar(SM::X_FULL), cc * 64, own0, b * p.Hkv + hk);
            tma_load_3d(sbase + SM::kX + SM::kTile + cc * (BT * 128), &tmV, bar(SM::X_FULL), cc * 64, own0, b * p.Hkv + hk);
          } else {
            tma_load_3d(sbase + SM::kX + cc * (BT * 128), &tmQ, bar(SM::X_FULL), cc * 64, own0, b * p.H + h0);
            tma_load_3d(sbase + SM::kX + SM::kTile + cc * (BT * 128), &tmdO, bar(SM::X_FULL), cc * 64, own0, b * p.H + h0);
          }
        }
      }
      bool ok = true;
      for (int n = 0; n < n_iter && ok; ++n) {
        const int s = n % kStages;
        const int g = (MODE == DKDV) ? n / it_n : 0;
        const int tile = it_lo + ((MODE == DKDV) ? n % it_n : n);
        const int row0 = tile * BT;
        if (n >= kStages)
          ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::Y_EMPTY + s), ((n / kStages) - 1) & 1, abort_flag, &g_attn_bwd_status, 101));
        if (!ok) break;
        if (lane == 0) {
          mbar_expect_tx(bar(SM::Y_FULL + s), 2 * SM::kTile);
          const uint32_t y1 = sbase + SM::kY + s * 2 * SM::kTile, y2 = y1 + SM::kTile;
#pragma unroll
          for (int cc = 0; cc < D / 64; ++cc) {
            if (MODE == DKDV) {
              tma_load_3d(y1 + cc * (BT * 128), &tmQ, bar(SM::Y_FULL + s), cc * 64, row0, b * p.H + h0 + g);
              tma_load_3d(y2 + cc * (BT * 128), &tmdO, bar(SM::Y_FULL + s), cc * 64, row0, b * p.H + h0 + g);
            } else {
              tma_load_3d(y1 + cc * (BT * 128), &tmK, bar(SM::Y_FULL + s), cc * 64, row0, b * p.Hkv + hk);
              tma_load_3d(y2 + cc * (BT * 128), &tmV, bar(SM::Y_FULL + s), cc * 64, row0, b * p.Hkv + hk);
            }
          }
        }
        // statistics / document ids of the streamed tile's positions
        float* slse = stat(s, 0); float* sdel = stat(s, 1); int* sdoc = reinterpret_cast<int*>(stat(s, 2));
        int dmin = 0x7fffffff, dmax = (int)0x80000000;
        for (int idx = lane; idx < BT; idx += 32) {
          const int row = row0 + idx;
          int doc = 0;
          if (MODE == DKDV) {
            const bool valid = row < q_lim;
            const size_t si = (size_t)(b * p.H + h0 + g) * p.Sq + (valid ? row : 0);
            // Both statistics are staged NEGATED, as the addends of the element pass's fused multiply-adds:
            // -lse2, and -Delta (with score mods) or -scale * Delta (without).
            slse[idx] = valid ? -lse2g[si] : -INFINITY;
            sdel[idx] = valid ? -deltag[si] * (p.score_flags != 0 ? 1.f : p.scale) : 0.f;
            if (p.mask_flags & TYLO_MASK_DOCUMENT) doc = p.doc_q[(size_t)b * p.doc_stride + min(row, p.Sq - 1) + p.input_pos];
          } else {
            if (p.mask_flags & TYLO_MASK_DOCUMENT) doc = p.doc_kv[(size_t)b * p.doc_stride + min(row, p.Sk - 1)];
          }
          sdoc[idx] = doc;
          dmin = min(dmin, doc); dmax = max(dmax, doc);
        }
        if (p.mask_flags & TYLO_MASK_DOCUMENT) {
          // smallest and largest id of the tile: equal means one document, which lets the compute
          // warps drop the per-element comparison or skip the tile
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            dmin = min(dmin, __shfl_xor_sync(0xffffffffu, dmin, o));
            dmax = max(dmax, __shfl_xor_sync(0xffffffffu, dmax, o));
          }
          if (lane == 0) { sdoc[BT] = dmin; sdoc[BT + 1] = dmax; }
        }
        mbar_arrive(bar(SM::STAT_FULL + s));
      }
    } else if (warp == 1 && lane == 0 && n_iter > 0) {
      // ------------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc_ss = idesc_f16(Fmt<T>::v, 0, 0, BT, BT);
      constexpr uint32_t idesc_ts = idesc_f16(Fmt<T>::v, 0, 1, BT, D);
      const uint64_t dk_hi = smem_desc_sw128(0, 16, 1024);            // K-major operand
      const uint64_t dmn_hi = smem_desc_sw128(0, BT * 128, 1024);     // MN-major operand
      auto desc_at = [](uint64_t hi, uint32_t saddr) { return hi | (uint64_t)((saddr & 0x3ffff) >> 4); };
      const uint32_t x1 = sbase + SM::kX, x2 = x1 + SM::kTile;
      auto issue_t1 = [&](int n) {     // T1 = X1 Y1^T  (S^T or S)
        const uint32_t y1 = sbase + SM::kY + (n % kStages) * 2 * SM::kTile;
        const uint64_t a1 = desc_at(dk_hi, x1), b1 = desc_at(dk_hi, y1);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = ((k / 4) * (BT * 128) + (k % 4) * 32) >> 4;
          mma_ss(tmem, a1 + off, b1 + off, idesc_ss, k > 0);
        }
        tc_commit(bar(SM::T1_FULL));
      };
      auto issue_t2 = [&](int n) {     // T2 = X2 Y2^T  (dP^T or dP)
        const uint32_t y2 = sbase + SM::kY + (n % kStages) * 2 * SM::kTile + SM::kTile;
        const uint64_t a2 = desc_at(dk_hi, x2), b2 = desc_at(dk_hi, y2);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = ((k / 4) * (BT * 128) + (k % 4) * 32) >> 4;
          mma_ss(tmem + 128, a2 + off, b2 + off, idesc_ss, k > 0);
        }
        tc_commit(bar(SM::T2_FULL));
      };
      auto issue_acc1 = [&](int n) {   // dV += P^T dO (DKDV only)
        const uint32_t y2 = sbase + SM::kY + (n % kStages) * 2 * SM::kTile + SM::kTile;
        const uint64_t b2 = desc_at(dmn_hi, y2);
#pragma unroll
        for (int k = 0; k < BT / 16; ++k)
          mma_ts(tmem + 256, tmem + (k / 4) * 64 + (k % 4) * 8, b2 + (uint32_t)((k * 2048) >> 4), idesc_ts, (n > 0) || (k > 0));
      };
      auto issue_acc2 = [&](int n) {   // dK += dS^T Q  /  dQ += dS K
        const uint32_t y1 = sbase + SM::kY + (n % kStages) * 2 * SM::kTile;
        const uint64_t b1 = desc_at(dmn_hi, y1);
#pragma unroll
        for (int k = 0; k < BT / 16; ++k)
          mma_ts(tmem + 384, tmem + 128 + (k / 4) * 64 + (k % 4) * 8, b1 + (uint32_t)((k * 2048) >> 4), idesc_ts, (n > 0) || (k > 0));
        tc_commit(bar(SM::Y_EMPTY + (n % kStages)));
      };
      bool ok = mbar_wait(bar(SM::X_FULL), 0, abort_flag, &g_attn_bwd_status, 201);
      ok = ok && mbar_wait(bar(SM::Y_FULL + 0), 0, abort_flag, &g_attn_bwd_status, 202);
      if (ok) { tc_fence_after(); issue_t1(0); issue_t2(0); }
      // Issue order per streamed tile n:  [U1(n) ready] acc1(n), T1(n+1)   [U2(n) ready] acc2(n), T2(n+1).
      // T1(n+1) only needs the T1 columns released (U1_FULL: P^T stored, or in DQ mode S read), so the
      // compute warps find the next S waiting when they finish tile n, while acc2(n) and T2(n+1) run.
      for (int n = 0; n < n_iter && ok; ++n) {
        ok = mbar_wait(bar(SM::U1_FULL), n & 1, abort_flag, &g_attn_bwd_status, 205);
        if (!ok) break;
        tc_fence_after();
        if (MODE == DKDV) issue_acc1(n);
        if (n + 1 < n_iter) {
          ok = mbar_wait(bar(SM::Y_FULL + (n + 1) % kStages), ((n + 1) / kStages) & 1, abort_flag, &g_attn_bwd_status, 204);
          if (!ok) break;
          tc_fence_after();
          issue_t1(n + 1);
        }
        ok = mbar_wait(bar(SM::U2_FULL), n & 1, abort_flag, &g_attn_bwd_status, 203);
        if (!ok) break;
        tc_fence_after();
        issue_acc2(n);
        if (n + 1 < n_iter) issue_t2(n + 1);
      }
      tc_commit(bar(SM::DONE));
      mbar_drain(bar(SM::DONE), 0);
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ------------------------------------------------------------------ compute warpgroups
    const int wg = (warp - 4) >> 2;                 // column half
    const int r = (warp & 3) * 32 + lane;           // TMEM lane = row of the owned tile
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const int own_row = own0 + r;
    const bool modded = p.score_flags != 0;
    const float c = p.scale * kLog2e;
    const float inv_cap = 1.f / p.cap;
    const bool has_doc = p.mask_flags & TYLO_MASK_DOCUMENT;
    // per-thread constants of the owned row
    float my_lse = -INFINITY, my_delta = 0.f, slope = 0.f;   // negated, like the staged per-column statistics
    int my_doc = 0;
    if (MODE == DQ) {
      if (own_row < q_lim) {
        const size_t si = (size_t)(b * p.H + h0) * p.Sq + own_row;
        my_lse = -lse2g[si]; my_delta = -deltag[si] * (modded ? 1.f : p.scale);
      }
      if (has_doc) my_doc = p.doc_q[(size_t)b * p.doc_stride + min(own_row, p.Sq - 1) + p.input_pos];
      if (p.score_flags & TYLO_SCORE_ALIBI) slope = p.slopes[h0];
    } else if (has_doc) {
      my_doc = p.doc_kv[(size_t)b * p.doc_stride + min(own_row, p.Sk - 1)];
    }
    const bool row_ok = (MODE == DKDV) ? (own_row < p.Sk) : (own_row < p.Sq);
    int iv_lo, iv_hi;
    const bool iv_any = row_interval(p, p.mask_flags, p.window, p.prefix_len, MODE == DKDV, own_row, k_len, q_lim, &iv_lo, &iv_hi);
    // OR-ed clauses of affine terms (mods.jl:164-167 in disjunctive normal form): one more interval of streamed
    // rows per clause; a pair is kept if any interval holds it.  (Clauses with a document term run on the
    // fp32-arithmetic kernels, see the dispatch.)
    const bool has_or = ORS && p.n_or > 0;
    // ALiBi slope gradient (mods.jl:296-303): the dQ kernel visits every (query, key, head) pair exactly
    // once, so it accumulates sum ds (q - kv) per thread and adds it to d_slopes[h] once per warp.
    const bool want_slope_grad = MODE == DQ && p.d_slopes != nullptr && (p.score_flags & TYLO_SCORE_ALIBI);
    float slope_acc = 0.f;
    // BiasScore (mods.jl:219-237, gradient :305-313): table (Sk, Sq, heads, batch) indexed by LOCAL rows, heads and
    // batch broadcast by modulo.  The dQ kernel owns a query row (its keys are contiguous in the table: 16-byte
    // loads and 16-byte reductions), the dK/dV kernel a key row (one entry per streamed query).  As with the slope
    // gradient the dQ kernel, which meets every pair once, adds dS at the bias's place in the chain to d_bias.
    const bool has_bias = (p.score_flags & TYLO_SCORE_BIAS) != 0;
    const bool want_bias_grad = MODE == DQ && has_bias && p.d_bias != nullptr;
    const bool bias_vec = (p.Sk & 3) == 0;
    size_t bias_row = 0;                 // dQ kernel: offset of this query row's entries in the table
    if (MODE == DQ && has_bias) bias_row = bias_index(p, b, h0, min(own_row, p.Sq - 1), 0);
    const unsigned iv_span = iv_any ? (unsigned)(iv_hi - iv_lo) : 0u;
    // soft cap: tanh(x) ~ x (1 - x^2/3 + 2x^4/15 - 17x^6/315) for |x| < 0.4, written in the raw dot product s (x = s k1)
    const float cap_k1 = p.scale * inv_cap, cap_k2 = p.cap * kLog2e, cap_u = cap_k1 * cap_k1;
    const float cap_b1 = -0.33333334f * cap_k1 * cap_u, cap_b2 = 0.13333334f * cap_k1 * cap_u * cap_u,
                cap_b3 = -0.05396825f * cap_k1 * cap_u * cap_u * cap_u;
    // the same constants as packed pairs for the two-columns-per-instruction forms
    const uint64_t c2 = pack_f32x2(c, c), scale2 = pack_f32x2(p.scale, p.scale), nscale2 = pack_f32x2(-p.scale, -p.scale);
    const uint64_t cb0_2 = pack_f32x2(cap_k1, cap_k1), cb1_2 = pack_f32x2(cap_b1, cap_b1), cb2_2 = pack_f32x2(cap_b2, cap_b2),
                   cb3_2 = pack_f32x2(cap_b3, cap_b3), ck2_2 = pack_f32x2(cap_k2, cap_k2);

    bool ok = true;
    for (int n = 0; n < n_iter && ok; ++n) {
      const int s = n % kStages;
      const int g = (MODE == DKDV) ? n / it_n : 0;
      const int tile0 = (it_lo + ((MODE == DKDV) ? n % it_n : n)) * BT;
      if (MODE == DKDV && (p.score_flags & TYLO_SCORE_ALIBI)) slope = p.slopes[h0 + g];
      const int qa = (MODE == DKDV) ? tile0 : own0, ka = (MODE == DKDV) ? own0 : tile0;
      bool partial = (ka + BT > k_len) || (qa + BT > q_lim) || (p.mask_flags & (TYLO_MASK_PREFIX | TYLO_MASK_PREFIX_LM));
      if (p.mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) partial = partial || (ka + BT - 1 > qa + p.input_pos);
      if (p.mask_flags & TYLO_MASK_SLIDING) partial = partial || (ka < qa + BT - 1 + p.input_pos - p.window);
      partial = partial || has_or;

      if (has_bias && n + 1 < n_iter) {
        // The next tile's block of the bias table, asked for a tile ahead so that it waits in L2: the element pass
        // reads it four entries at a time and would otherwise sit out a DRAM round trip for each.  dQ: this query
        // row's 128 entries (four lines); dK/dV: the line of this warp's 32 keys for each of the 128 queries,
        // four per lane.
        const int n1 = n + 1;
        const int t1 = (it_lo + ((MODE == DKDV) ? n1 % it_n : n1)) * BT;
        if (MODE == DQ) {
          const float* bn = p.bias + bias_row + min(t1, p.Sk - 1);
#pragma unroll
          for (int cl = 0; cl < 4; ++cl)
            if (t1 + cl * 32 < p.Sk) asm volatile("prefetch.global.L2 [%0];" ::"l"(bn + cl * 32));
        } else {
          const int g1 = n1 / it_n, kvb = min(own_row, p.Sk - 1);
#pragma unroll
          for (int cl = 0; cl < 4; ++cl) {
            const int qn = t1 + cl * 32 + lane;
            if (qn < p.Sq) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.bias + bias_index(p, b, h0 + g1, qn, kvb)));
          }
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::STAT_FULL + s), (n / kStages) & 1, abort_flag, &g_attn_bwd_status, 301));
      ok = ok && __all_sync(0xffffffffu, mbar_wait(bar(SM::T1_FULL), n & 1, abort_flag, &g_attn_bwd_status, 302));
      if (!ok) break;
      tc_fence_after();
      // Document mask: the producer left the smallest and largest id of the streamed tile.  One document
      // that none of this warp's 32 rows belongs to: P = dS = 0 for the warp's rows, nothing to compute.
      // One document that all of them belong to: no per-element comparison.
      bool doc_cmp = false;
      if (has_doc) {
        const int* sd = reinterpret_cast<const int*>(smem + SM::kStats + s * SM::kStatStage + 2 * BT * 4);
        const int dmin = sd[BT], dmax = sd[BT + 1];
        const bool one_doc = dmin == dmax;
        if (one_doc && __all_sync(0xffffffffu, my_doc != dmin)) {
          uint32_t z[16];
#pragma unroll
          for (int t = 0; t < 16; ++t) z[t] = 0u;
          if (MODE == DKDV) {
            tmem_st16x(tmem + lane_off + 64 * wg, z); tmem_st16x(tmem + lane_off + 64 * wg + 16, z);
            tc_wait_st();
          }
          tc_fence_before();
          mbar_arrive(bar(SM::U1_FULL));
          ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::T2_FULL), n & 1, abort_flag, &g_attn_bwd_status, 303));
          if (!ok) break;
          tc_fence_after();
          tmem_st16x(tmem + 128 + lane_off + 64 * wg, z); tmem_st16x(tmem + 128 + lane_off + 64 * wg + 16, z);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(SM::U2_FULL));
          continue;
        }
        doc_cmp = !(one_doc && __all_sync(0xffffffffu, my_doc == dmin));
        partial = partial || doc_cmp;
      }
      uint32_t sv[2][32], dv[2][32];
      tmem_ld32(tmem + lane_off + 64 * wg, sv[0]); tmem_ld32(tmem + lane_off + 64 * wg + 32, sv[1]);
      tc_wait_ld();
      const uint32_t stat_u = sbase + SM::kStats + s * SM::kStatStage;   // lse2[128], delta[128], doc[128]
      // column j of this warpgroup's half (streamed row tile0 + 64*wg + j) is inside the row's interval
      // iff (unsigned)(j - rel) <= iv_span; a row that pairs with nothing gets an unreachable start
      const int rel = iv_any ? iv_lo - tile0 - 64 * wg : 0x40000000;
      // (worked out per tile, and only when there are clauses, so that they cost the other paths no registers)
      int or_rel[kMaxOrClauses]; unsigned or_span[kMaxOrClauses];
      if (has_or) {
#pragma unroll
        for (int ci = 0; ci < kMaxOrClauses; ++ci) {
          or_rel[ci] = 0x40000000; or_span[ci] = 0u;
          if (ci < p.n_or) {
            int lo, hi;
            const MaskClause& cl = p.or_clause[ci];
            if (row_interval(p, cl.flags, cl.window, cl.prefix_len, MODE == DKDV, own_row, k_len, q_lim, &lo, &hi)) {
              or_rel[ci] = lo - tile0 - 64 * wg; or_span[ci] = (unsigned)(hi - lo);
            }
          }
        }
      }
      // the element passes exist in three forms: whole tile unmasked (0), one interval per row (1), the interval
      // plus those of the OR-ed clauses (2)
      auto keep_at = [&](int j, auto ors_c) -> bool {
        bool k = (unsigned)(j - rel) <= iv_span;
        if (decltype(ors_c)::value) {
#pragma unroll
          for (int ci = 0; ci < kMaxOrClauses; ++ci) k = k || ((unsigned)(j - or_rel[ci]) <= or_span[ci]);
        }
        return k;
      };
      using Lvl0 = std::integral_constant<int, 0>; using Lvl1 = std::integral_constant<int, 1>;
      using Lvl2 = std::integral_constant<int, 2>;
      // position difference q - kv of column j: dpos + j in DKDV mode, dpos - j in DQ mode
      const int dpos = (MODE == DKDV) ? tile0 + 64 * wg + p.input_pos - own_row : own_row + p.input_pos - tile0 - 64 * wg;
      const float fdpos = (float)dpos;

      // Each warpgroup writes its packed 16-bit columns over the first half of ITS OWN 64 T columns
      // (the MMA addresses the two 32-column pieces separately), so no thread overwrites T values
      // another thread has yet to read and the two warpgroups need no rendezvous.
      if (!modded) {
        // pass 1 (while the dP MMAs run): p = exp2(c s - lse2), masked; kept in fp32 over sv
        auto pass_p = [&](auto partial_c) {
          constexpr bool PART = decltype(partial_c)::value != 0;
          using ORS = std::bool_constant<decltype(partial_c)::value == 2>;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            uint32_t up[16];
#pragma unroll
            for (int t = 0; t < 32; t += 4) {
              const int col0 = 64 * wg + q * 32 + t;
              float l0 = my_lse, l1 = my_lse, l2 = my_lse, l3 = my_lse;
              int d0 = 0, d1 = 0, d2 = 0, d3 = 0;
              if (MODE == DKDV) lds128(stat_u + col0 * 4, l0, l1, l2, l3);
              if (PART) lds128i(stat_u + 2 * BT * 4 + col0 * 4, d0, d1, d2, d3);
              const float lse4[4] = {l0, l1, l2, l3};
              const int doc4[4] = {d0, d1, d2, d3};
              float pp[4];
#pragma unroll
              for (int e = 0; e < 4; e += 2) {     // exponent arguments two at a time: s c + (-lse2)
                float x0, x1;
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[q][t + e]), __uint_as_float(sv[q][t + e + 1])), c2,
                                       pack_f32x2(lse4[e], lse4[e + 1])), x0, x1);
                pp[e] = ex2(x0); pp[e + 1] = ex2(x1);
              }
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (PART) {
                  const int j = q * 32 + t + e;
                  bool keep = keep_at(j, ORS{});
                  if (doc_cmp) keep = keep && (doc4[e] == my_doc);
                  if (!keep) pp[e] = 0.f;
                }
                sv[q][t + e] = __float_as_uint(pp[e]);
              }
              up[t / 2] = pack16<T>(pp[0], pp[1]); up[t / 2 + 1] = pack16<T>(pp[2], pp[3]);
            }
            if (MODE == DKDV) tmem_st16x(tmem + lane_off + 64 * wg + q * 16, up);
          }
        };
        if (!partial) pass_p(Lvl0{}); else if (!has_or) pass_p(Lvl1{}); else pass_p(Lvl2{});
        if (MODE == DKDV) tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(SM::U1_FULL));       // T1 columns released: dV's MMAs / the next S may start
        ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::T2_FULL), n & 1, abort_flag, &g_attn_bwd_status, 303));
        if (!ok) break;
        tc_fence_after();
        tmem_ld32(tmem + 128 + lane_off + 64 * wg, dv[0]); tmem_ld32(tmem + 128 + lane_off + 64 * wg + 32, dv[1]);
        tc_wait_ld();
        // pass 2: ds = p (dp - delta) * scale
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          uint32_t ud[16];
#pragma unroll
          for (int t = 0; t < 32; t += 4) {
            const int col0 = 64 * wg + q * 32 + t;
            float e0 = my_delta, e1 = my_delta, e2 = my_delta, e3 = my_delta;
            if (MODE == DKDV) lds128(stat_u + BT * 4 + col0 * 4, e0, e1, e2, e3);
            const float del4[4] = {e0, e1, e2, e3};
            float dd[4];
#pragma unroll
            for (int e = 0; e < 4; e += 2) {      // p (dp scale + (-scale Delta)), two at a time
              const uint64_t g2 = fma_f32x2(pack_f32x2(__uint_as_float(dv[q][t + e]), __uint_as_float(dv[q][t + e + 1])), scale2,
                                            pack_f32x2(del4[e], del4[e + 1]));
              unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(sv[q][t + e]), __uint_as_float(sv[q][t + e + 1])), g2),
                           dd[e], dd[e + 1]);
            }
            ud[t / 2] = pack16<T>(dd[0], dd[1]); ud[t / 2 + 1] = pack16<T>(dd[2], dd[3]);
          }
          tmem_st16x(tmem + 128 + lane_off + 64 * wg + q * 16, ud);
        }
      } else {
        // score mods: p and the VJP factor come out of one evaluation, so both T tiles are awaited first
        ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::T2_FULL), n & 1, abort_flag, &g_attn_bwd_status, 303));
        if (!ok) break;
        tc_fence_after();
        tmem_ld32(tmem + 128 + lane_off + 64 * wg, dv[0]); tmem_ld32(tmem + 128 + lane_off + 64 * wg + 32, dv[1]);
        tc_wait_ld();
        // Soft cap alone with every score of the warp small against the cap (the usual case): tanh is
        // an odd polynomial with the constants folded in, branch-free, one SFU operation per element.
        bool fastcap = false;
        if (p.score_flags == TYLO_SCORE_SOFTCAP) {
          float am0 = 0.f, am1 = 0.f;
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            am0 = fmaxf(am0, fabsf(__uint_as_float(sv[0][t])));
            am1 = fmaxf(am1, fabsf(__uint_as_float(sv[1][t])));
          }
          fastcap = __all_sync(0xffffffffu, fmaxf(am0, am1) * cap_k1 < 0.4f);
        }
        auto run = [&](auto partial_c, auto fast_c) {
          constexpr bool PART = decltype(partial_c)::value != 0;
          using ORS = std::bool_constant<decltype(partial_c)::value == 2>;
          // kind of score-mod evaluation: 0 the general chain, 1 soft cap alone with small scores (polynomial), 2 additive
          // mods only (ALiBi, bias table): one exponent per element, no run-time flag tests, no conversions
          constexpr int KIND = decltype(fast_c)::value;
          constexpr bool FAST = KIND == 1;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            uint32_t up[16], ud[16];
#pragma unroll
            for (int t = 0; t < 32; t += 4) {
              const int col0 = 64 * wg + q * 32 + t;
              float l0 = my_lse, l1 = my_lse, l2 = my_lse, l3 = my_lse, e0 = my_delta, e1 = my_delta, e2 = my_delta, e3 = my_delta;
              int d0 = 0, d1 = 0, d2 = 0, d3 = 0;
              if (MODE == DKDV) {
                lds128(stat_u + col0 * 4, l0, l1, l2, l3);
                lds128(stat_u + BT * 4 + col0 * 4, e0, e1, e2, e3);
              }
              if (PART) lds128i(stat_u + 2 * BT * 4 + col0 * 4, d0, d1, d2, d3);
              const float lse4[4] = {l0, l1, l2, l3}, del4[4] = {e0, e1, e2, e3};
              const int doc4[4] = {d0, d1, d2, d3};
              float pp[4], dd[4];
              if (FAST) {
                // t = tanh(s k1) = s (b0 + u (b1 + u (b2 + u b3))), u = s^2;  modded score cap*t;  VJP factor
                // scale (1 - t^2); two columns per instruction
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                  const uint64_t s2 = pack_f32x2(__uint_as_float(sv[q][t + e]), __uint_as_float(sv[q][t + e + 1]));
                  const uint64_t u2 = mul_f32x2(s2, s2);
                  const uint64_t th2 = mul_f32x2(s2, fma_f32x2(u2, fma_f32x2(u2, fma_f32x2(u2, cb3_2, cb2_2), cb1_2), cb0_2));
                  float x0, x1;
                  unpack_f32x2(fma_f32x2(th2, ck2_2, pack_f32x2(lse4[e], lse4[e + 1])), x0, x1);
                  float p0 = ex2(x0), p1 = ex2(x1);
                  if (PART) {
                    const int j = q * 32 + t + e;
                    bool k0 = keep_at(j, ORS{}), k1 = keep_at(j + 1, ORS{});
                    if (doc_cmp) { k0 = k0 && (doc4[e] == my_doc); k1 = k1 && (doc4[e + 1] == my_doc); }
                    if (!k0) p0 = 0.f;
                    if (!k1) p1 = 0.f;
                  }
                  pp[e] = p0; pp[e + 1] = p1;
                  const uint64_t f2 = fma_f32x2(mul_f32x2(th2, nscale2), th2, scale2);          // scale - scale t^2
                  const uint64_t g2 = add_f32x2(pack_f32x2(__uint_as_float(dv[q][t + e]), __uint_as_float(dv[q][t + e + 1])),
                                                pack_f32x2(del4[e], del4[e + 1]));                 // dp + (-Delta)
                  unpack_f32x2(mul_f32x2(mul_f32x2(pack_f32x2(p0, p1), g2), f2), dd[e], dd[e + 1]);
                }
              } else {
                float bias4[4] = {0.f, 0.f, 0.f, 0.f}, dsa[4];
                const int scol = tile0 + col0;        // first of the four streamed rows (keys for dQ, queries for dK/dV)
                if (has_bias) {
                  if (MODE == DQ) {
                    const float* bp = p.bias + bias_row + scol;
                    if (bias_vec && scol + 3 < p.Sk) {
                      const float4 f = __ldg(reinterpret_cast<const float4*>(bp));
                      bias4[0] = f.x; bias4[1] = f.y; bias4[2] = f.z; bias4[3] = f.w;
                    } else {
#pragma unroll
                      for (int e = 0; e < 4; ++e) bias4[e] = (scol + e < p.Sk) ? __ldg(bp + e) : 0.f;
                    }
                  } else {
                    const int kvb = min(own_row, p.Sk - 1);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                      bias4[e] = __ldg(p.bias + bias_index(p, b, h0 + g, min(scol + e, p.Sq - 1), kvb));
                  }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const int j = q * 32 + t + e;
                  bool keep = keep_at(j, ORS{});
                  if (PART && doc_cmp) keep = keep && (doc4[e] == my_doc);
                  if (KIND == 2) {
                    // exponent = s c + (slope (q - kv) + bias) log2e - lse2;  dS at the mods' place = p (dP - Delta)
                    const float pos = (MODE == DKDV) ? fdpos + (float)j : fdpos - (float)j;
                    float pv = ex2(fmaf(__uint_as_float(sv[q][t + e]), c, fmaf(fmaf(slope, pos, bias4[e]), kLog2e, lse4[e])));
                    if (PART && !keep) pv = 0.f;
                    dsa[e] = pv * (__uint_as_float(dv[q][t + e]) + del4[e]);
                    dd[e] = dsa[e] * p.scale;
                    pp[e] = pv;
                    if (MODE == DQ && want_slope_grad) slope_acc = fmaf(dsa[e], pos, slope_acc);
                  } else {
                    const int qmk = (MODE == DKDV) ? dpos + j : dpos - j;
                    pp[e] = element<true, PART>(p, c, slope, inv_cap, __uint_as_float(sv[q][t + e]), __uint_as_float(dv[q][t + e]),
                                                lse4[e], del4[e], qmk, keep, bias4[e], dd[e], dsa[e]);
                    if (MODE == DQ && want_slope_grad) slope_acc = fmaf(dsa[e], (float)qmk, slope_acc);
                  }
                }
                if (MODE == DQ && want_bias_grad && own_row < p.Sq) {
                  // masked pairs and keys beyond the length have p = 0, hence dS = 0: nothing to add there
                  float* gp = p.d_bias + bias_row + scol;
                  if (bias_vec && scol + 3 < p.Sk) {
                    if (dsa[0] != 0.f || dsa[1] != 0.f || dsa[2] != 0.f || dsa[3] != 0.f)
                      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gp), "f"(dsa[0]), "f"(dsa[1]), "f"(dsa[2]),
                                   "f"(dsa[3]) : "memory");
                  } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                      if (scol + e < p.Sk && dsa[e] != 0.f) atomicAdd(gp + e, dsa[e]);
                  }
                }
              }
              up[t / 2] = pack16<T>(pp[0], pp[1]); up[t / 2 + 1] = pack16<T>(pp[2], pp[3]);
              ud[t / 2] = pack16<T>(dd[0], dd[1]); ud[t / 2 + 1] = pack16<T>(dd[2], dd[3]);
            }
            if (MODE == DKDV) tmem_st16x(tmem + lane_off + 64 * wg + q * 16, up);
            tmem_st16x(tmem + 128 + lane_off + 64 * wg + q * 16, ud);
          }
        };
        if (fastcap) {
          if (!partial) run(Lvl0{}, Lvl1{}); else if (!has_or) run(Lvl1{}, Lvl1{}); else run(Lvl2{}, Lvl1{});
        } else if (!(p.score_flags & (TYLO_SCORE_SOFTCAP | TYLO_SCORE_SOFTCAP_FIRST))) {
          if (!partial) run(Lvl0{}, Lvl2{}); else if (!has_or) run(Lvl1{}, Lvl2{}); else run(Lvl2{}, Lvl2{});
        } else {
          if (!partial) run(Lvl0{}, Lvl0{}); else if (!has_or) run(Lvl1{}, Lvl0{}); else run(Lvl2{}, Lvl0{});
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(SM::U1_FULL));
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(SM::U2_FULL));
    }

    if (want_slope_grad && ok) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) slope_acc += __shfl_xor_sync(0xffffffffu, slope_acc, o);
      if (lane == 0 && slope_acc != 0.f) atomicAdd(p.d_slopes + h0, slope_acc);
    }

    // ---- epilogue: this warpgroup stores columns [wg*D/2, (wg+1)*D/2) of each accumulator
    if (n_iter > 0 && ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::DONE), 0, abort_flag, &g_attn_bwd_status, 304));
      tc_fence_after();
    }
    if (ok) {
      constexpr int HALF = D / 2;
      const size_t orow = (MODE == DKDV) ? ((size_t)(b * p.Hkv + hk) * p.Sk + (row_ok ? own_row : 0))
                                         : ((size_t)(b * p.H + h0) * p.Sq + (row_ok ? own_row : 0));
#pragma unroll
      for (int a = (MODE == DKDV ? 0 : 1); a < 2; ++a) {
        // (a head dim below the tile's runs zero-padded: rows are p.Dk long, columns beyond are not stored)
        T* dst = ((MODE == DKDV) ? (a == 0 ? out1 : out2) : out1) + orow * p.Dk + wg * HALF;
#pragma unroll
        for (int q = 0; q < HALF / 32; ++q) {
          uint32_t acc[32];
          if (n_iter > 0) { tmem_ld32(tmem + 256 + a * 128 + lane_off + wg * HALF + q * 32, acc); tc_wait_ld(); }
          uint4 o4[4];
          uint32_t* ow = reinterpret_cast<uint32_t*>(o4);
#pragma unroll
          for (int t = 0; t < 16; ++t)
            ow[t] = (n_iter > 0) ? pack16<T>(__uint_as_float(acc[2 * t]), __uint_as_float(acc[2 * t + 1])) : 0u;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v)
              if (wg * HALF + q * 32 + v * 8 < p.Dk) *reinterpret_cast<uint4*>(dst + q * 32 + v * 8) = o4[v];
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0 && lane == 0 && n_iter > 0) {
    mbar_drain(bar(SM::X_FULL), 0);
    for (int s = 0; s < kStages && s < n_iter; ++s) {
      const int last = ((n_iter - 1 - s) / kStages) * kStages + s;
      mbar_drain(bar(SM::Y_FULL + s), (last / kStages) & 1);
    }
  }
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// Delta[row] = sum_d dO*O and lse2[row] = log2-domain log-sum-exp from the forward's (M, L).
// LPR = Dv / 8 lanes share a row (one 16-byte packet each), so a warp covers 32 / LPR rows.
template <typename T, int LPR>
__global__ void __launch_bounds__(256)
bwd_prep_kernel(float* __restrict__ Delta, float* __restrict__ lse2, const T* __restrict__ O,
                const T* __restrict__ dO, const float* __restrict__ M, const float* __restrict__ L,
                long long rows, int natural_stats, int Dr) {
  // Dr: the rows' real length (a multiple of 8, at most LPR * 8)
  constexpr int RPW = 32 / LPR;
  const int lane = threadIdx.x & 31;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW + lane / LPR;
  const int sub = lane % LPR;
  float s = 0.f;
  if (row < rows && sub * 8 < Dr) {
    Pack<T> a, b2;
    a.raw = ld_stream(O + (size_t)row * Dr + sub * 8);
    b2.raw = ld_stream(dO + (size_t)row * Dr + sub * 8);
    float fa[8], fb[8];
    a.unpack(fa); b2.unpack(fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += fa[j] * fb[j];
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (sub == 0 && row < rows) {
    Delta[row] = s;
    const float l = L[row], m = M[row];
    lse2[row] = (l > 0.f) ? (natural_stats ? m * kLog2e : m) + log2f(l) : INFINITY;
  }
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

static int32_t make_tmap(CUtensorMap* map, const void* base, int D, int S, int BH) {
  auto fn = encode_fn();
  TYLO_REQUIRE(fn, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)S * D * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)BT, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TYLO_REQUIRE(r == CUDA_SUCCESS, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TYLO_OK;
}

template <typename T, int D>
static int32_t launch(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V, const void* O,
                      const void* dO, const float* M, const float* L, float* Delta, float* lse2, const AttnParams& p,
                      cudaStream_t st) {
  const long long rows = (long long)p.Sq * p.H * p.B;
  constexpr int LPR = D / 8, RPB = 8 * (32 / LPR);   // lanes per row, rows per 256-thread block
  bwd_prep_kernel<T, LPR><<<(unsigned)((rows + RPB - 1) / RPB), 256, 0, st>>>(Delta, lse2, (const T*)O, (const T*)dO, M, L,
                                                                             rows, p.natural_stats, p.Dk);
  if (int32_t rc = check_launch("attn_bwd_prep")) return rc;
  CUtensorMap mq, mk, mv, mdo;
  // the maps describe the arrays as they are (rows of p.Dk elements); boxes reaching beyond read zeros
  if (int32_t rc = make_tmap(&mq, Q, p.Dk, p.Sq, p.H * p.B)) return rc;
  if (int32_t rc = make_tmap(&mk, K, p.Dk, p.Sk, p.Hkv * p.B)) return rc;
  if (int32_t rc = make_tmap(&mv, V, p.Dk, p.Sk, p.Hkv * p.B)) return rc;
  if (int32_t rc = make_tmap(&mdo, dO, p.Dk, p.Sq, p.H * p.B)) return rc;
  const bool ors = p.n_or > 0;
  {
    auto kern = ors ? attn_bwd_sm100_kernel<T, D, DKDV, true> : attn_bwd_sm100_kernel<T, D, DKDV, false>;
    TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::kDynamic));
    const long long grid = (long long)((p.Sk + BT - 1) / BT) * p.Hkv * p.B;
    kern<<<(unsigned)grid, kThreads, Smem<D>::kDynamic, st>>>(mq, mk, mv, mdo, (T*)dV, (T*)dK, lse2, Delta, p);
    if (int32_t rc = check_launch("attn_bwd_sm100<dkdv>")) return rc;
  }
  {
    auto kern = ors ? attn_bwd_sm100_kernel<T, D, DQ, true> : attn_bwd_sm100_kernel<T, D, DQ, false>;
    TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<D>::kDynamic));
    const long long grid = (long long)((p.Sq + BT - 1) / BT) * p.H * p.B;
    // The dQ kernel reads nothing the dK/dV kernel writes (both depend only on the inputs and on the prep
    // kernel, which finished before the dK/dV kernel started).  It is launched as a programmatic
    // dependent of the dK/dV kernel and never waits on it, so its CTAs fill the SMs that the last wave
    // of the dK/dV kernel leaves idle.  Work submitted to the stream afterwards still waits for both.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = Smem<D>::kDynamic; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    TYLO_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, mdo, (T*)dQ, (T*)nullptr, (const float*)lse2,
                                    (const float*)Delta, p));
    if (int32_t rc = check_launch("attn_bwd_sm100<dq>")) return rc;
  }
  return TYLO_OK;
}

}  // namespace bwd

bool attn_bwd_sm100_supported(const AttnParams& p, int32_t dtype) {
  if (dtype != TYLO_BF16 && dtype != TYLO_F16) return false;
  if (p.Dk != p.Dv || p.Dk < 8 || p.Dk % 8 != 0 || p.Dk > 128) return false;     // below 64 / 128: zero-padded
  if ((long long)p.Sq * p.H * p.B > 0x7fffffffLL / 2 || (long long)p.Sk * p.Hkv * p.B > 0x7fffffffLL / 2) return false;
  return true;
}

int64_t attn_bwd_sm100_workspace_bytes(int Sq, int H, int B) {
  const int64_t n = (int64_t)Sq * H * B * 4;
  return (n + 255) / 256 * 256;
}

int32_t attn_bwd_sm100(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V, const void* O,
                       const void* dO, const float* M, const float* L, float* Delta, void* workspace,
                       const AttnParams& p, int32_t dtype, cudaStream_t st) {
  float* lse2 = static_cast<float*>(workspace);
  if (dtype == TYLO_BF16) {
    if (p.Dk > 64) return bwd::launch<__nv_bfloat16, 128>(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, lse2, p, st);
    return bwd::launch<__nv_bfloat16, 64>(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, lse2, p, st);
  }
  if (p.Dk > 64) return bwd::launch<__half, 128>(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, lse2, p, st);
  return bwd::launch<__half, 64>(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, lse2, p, st);
}


int32_t attn_bwd_sm100_status(int* out) {
  int v = 0;
  TYLO_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn_bwd_status, sizeof(int)));
  *out = v;
  if (v != 0) {
    const int zero = 0;
    TYLO_CUDA_OK(cudaMemcpyToSymbol(g_attn_bwd_status, &zero, sizeof(int)));
  }
  return TYLO_OK;
}

}  // namespace tylo
