// Flash-attention forward for sm_100a: tcgen05.mma with accumulators in tensor memory, operands
// staged by TMA into a 128-byte-swizzled shared-memory ring, warp-specialised roles.
//
// One CTA owns 256 query rows of one (head, batch) as two 128-row tiles A and B, and walks the
// 128-key tiles their masks allow.  The two tiles share every K/V tile and ping-pong on the
// tensor pipe: while the softmax warpgroup of one tile works, the MMA issuer runs the other's.
//
//   warp 0       TMA producer: Q_A, Q_B once, then K and V tiles through rings (mbarrier full/empty).
//   warp 1       MMA issuer (one elected lane), owner of the tensor-memory allocation:
//                  S_X  = Q_X K_j^T       (both operands from shared memory, 128 x 128 x D)
//                  O_X += P_X V_j         (P from tensor memory, V MN-major from shared memory)
//   warps 4..7   softmax of tile A, warps 8..11 softmax of tile B: thread r owns query row r
//                (= TMEM lane r).  Reads S with tcgen05.ld, applies score/mask mods, keeps a running
//                max / sum in fp32, writes P (bf16/f16) back over the S columns with tcgen05.st,
//                rescales O in TMEM only when the row max grew by more than 2^8 (lazy rescaling),
//                and writes the final O, M, L.
//   warps 2,3    idle (they only donate their registers to the softmax warpgroups).
//
// TMEM columns: [0,128) S_A/P_A, [128,256) S_B/P_B, [256,256+D) O_A, [384,384+D) O_B.
// No multicast, no clusters.  Every mbarrier wait is bounded; a time-out sets a status word and
// the CTA drains instead of hanging.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <type_traits>

#include "attn_dispatch.cuh"
#include "sm100_ptx.cuh"

namespace tylo {
using namespace sm100;

__device__ int g_attn_fwd_status = 0;

constexpr uint32_t kRuntimeMods = 0x80000000u;  // template value: read the flags from AttnParams
constexpr int BM = 128, BN = 128;               // rows of one Q tile, keys of one K/V tile
constexpr int kFwdThreads = 384;

template <int D> struct FwdSmem {
  static constexpr int kStages = (D == 128) ? 2 : 4;
  static constexpr int kTile = BM * D * 2;             // bytes of one Q / K / V tile
  static constexpr int kQ = 0;                          // two Q tiles
  static constexpr int kK = 2 * kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kBars = kV + kStages * kTile;    // 8-byte mbarriers
  static constexpr int Q_FULL = 0, K_FULL = 2, K_EMPTY = K_FULL + kStages, V_FULL = K_EMPTY + kStages,
                       V_EMPTY = V_FULL + kStages, S_FULL = V_EMPTY + kStages, P_FULL = S_FULL + 2,
                       O_READY = P_FULL + 2, DONE = O_READY + 2, kNumBars = DONE + 1;
  static constexpr int kMisc = kBars + 8 * kNumBars;    // tmem base, abort flag
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;        // slack for manual 1024-byte alignment
};

template <typename T> struct MmaFmt;
template <> struct MmaFmt<__nv_bfloat16> { static constexpr int v = 1; };
template <> struct MmaFmt<__half> { static constexpr int v = 0; };

template <typename T> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// cap * tanh(s / cap): odd polynomial on the FMA pipe for small arguments (the common case for a
// soft cap well above the score range), hardware tanh otherwise.
__device__ __forceinline__ float softcap(float s, float cap, float inv_cap) {
  const float x = s * inv_cap, x2 = x * x;
  float t;
  if (x2 < 0.16f) {
    t = x * fmaf(x2, fmaf(x2, fmaf(x2, -0.05396825f, 0.13333334f), -0.33333334f), 1.f);
  } else {
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  }
  return cap * t;
}

struct TileRange { int s, e; };  // CTA-local key-tile indices [s, e) a Q tile takes part in

// Softmax / epilogue of one Q tile (one warpgroup, 128 threads).
template <typename T, int D, uint32_t MASK, uint32_t SCORE>
__device__ __forceinline__ void softmax_tile(const AttnParams& p, const uint32_t mask_flags,
                                             const uint32_t score_flags, const int X, const int q0x, const int jlo,
                                             const TileRange tr, const int b, const int h, const uint32_t tmem,
                                             const uint32_t sbase, volatile int* abort_flag, T* __restrict__ O,
                                             float* __restrict__ Mout, float* __restrict__ Lout, const int k_len,
                                             const int q_lim) {
  // k_len: keys of this batch entry that exist (<= Sk); q_lim: rows below it are computed and stored
  using SM = FwdSmem<D>;
  auto bar = [&](int i) { return sbase + SM::kBars + 8 * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wq = warp & 3;                       // TMEM lane quarter this warp may touch
  const int r = wq * 32 + lane;                  // row within the tile
  const int row = q0x + r, qpos = row + p.input_pos;
  const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
  const uint32_t ts = tmem + lane_off + X * 128;
  const uint32_t to = tmem + lane_off + 256 + X * 128;
  const bool modded = score_flags != 0;
  // units of the running max: raw dot products when there is no score mod (c folds the scale),
  // log2-scaled modded scores otherwise
  const float c = modded ? 1.f : p.scale * kLog2e;
  const float slope = (score_flags & TYLO_SCORE_ALIBI) ? p.slopes[h] : 0.f;
  const float inv_cap = 1.f / p.cap;
  int my_doc = 0;
  if (mask_flags & TYLO_MASK_DOCUMENT) my_doc = p.doc_q[(size_t)b * p.doc_stride + min(qpos, (int)p.Sq - 1 + p.input_pos)];
  const int n = tr.e - tr.s;

  // Every mask term except an element-wise document comparison keeps ONE interval of keys per row:
  // [row_lo, row_hi] (mods.jl:101-167 reduced to bounds).  Inside a tile the test is then one unsigned
  // compare per element against the tile-relative start.
  int row_lo = 0, row_hi = k_len - 1;
  if (mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) row_hi = min(row_hi, qpos);
  if (mask_flags & TYLO_MASK_SLIDING) row_lo = max(row_lo, qpos - p.window);
  if (mask_flags & TYLO_MASK_PREFIX) row_hi = min(row_hi, p.prefix_len - 1);
  if (mask_flags & TYLO_MASK_PREFIX_LM) row_hi = min(row_hi, max(qpos, p.prefix_len - 1));
  const bool row_any = row_hi >= row_lo;
  const unsigned row_span = row_any ? (unsigned)(row_hi - row_lo) : 0u;
  // soft cap as s * P(s^2) with the constants of the tanh series folded in (see below)
  const float cap_k1 = p.scale * inv_cap;
  const float cap_a0 = cap_k1 * p.cap * kLog2e, cap_u = cap_k1 * cap_k1;
  const float cap_a1 = -0.33333334f * cap_a0 * cap_u, cap_a2 = 0.13333334f * cap_a0 * cap_u * cap_u,
              cap_a3 = -0.05396825f * cap_a0 * cap_u * cap_u * cap_u;

  float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
  bool ok = true;
  for (int i = 0; i < n && ok; ++i) {
    const int kv0 = (jlo + tr.s + i) * BN;
    int ids[4] = {0, 0, 0, 0};   // document ids of the tile's keys: lane t holds key q*32 + t
    bool doc_uniform = false;
    if (mask_flags & TYLO_MASK_DOCUMENT) {
#pragma unroll
      for (int q = 0; q < 4; ++q) ids[q] = p.doc_kv[(size_t)b * p.doc_stride + min(kv0 + q * 32 + lane, p.Sk - 1)];
      const int id0 = __shfl_sync(0xffffffffu, ids[0], 0);
      doc_uniform = __all_sync(0xffffffffu, ids[0] == id0 && ids[1] == id0 && ids[2] == id0 && ids[3] == id0);
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::S_FULL + X), i & 1, abort_flag, &g_attn_fwd_status, 301));
    if (!ok) break;
    tc_fence_after();
    // P = 0 for the whole tile: nothing to load, exponentiate or rescale
    auto pass_empty_tile = [&]() {
      uint32_t z[32];
#pragma unroll
      for (int t = 0; t < 32; ++t) z[t] = 0u;
      tmem_st32(ts, z); tmem_st32(ts + 32, z);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(SM::P_FULL + X));
    };
    if ((mask_flags & TYLO_MASK_DOCUMENT) && doc_uniform && __all_sync(0xffffffffu, ids[0] != my_doc)) {
      // all 128 keys belong to one document that none of this warp's 32 rows belongs to
      pass_empty_tile();
      continue;
    }
    uint32_t sr[4][32];
#pragma unroll
    for (int q = 0; q < 4; ++q) tmem_ld32(ts + q * 32, sr[q]);
    tc_wait_ld();

    // which tiles need the element-wise mask?
    const int q_lo = q0x + p.input_pos, q_hi = q0x + BM - 1 + p.input_pos;
    bool partial = kv0 + BN > k_len;
    if (mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING | TYLO_MASK_PREFIX_LM)) partial = partial || (kv0 + BN - 1 > q_lo);
    if (mask_flags & TYLO_MASK_SLIDING) partial = partial || (kv0 < q_hi - p.window);
    if (mask_flags & (TYLO_MASK_PREFIX | TYLO_MASK_PREFIX_LM)) partial = true;
    if (mask_flags & TYLO_MASK_DOCUMENT) partial = partial || !doc_uniform || __any_sync(0xffffffffu, ids[0] != my_doc);
    const bool doc_elementwise = (mask_flags & TYLO_MASK_DOCUMENT) && !doc_uniform;
    const bool row_doc_ok = !(mask_flags & TYLO_MASK_DOCUMENT) || doc_elementwise || (__shfl_sync(0xffffffffu, ids[0], 0) == my_doc);

    // score mods (compile-time selected), then the element-wise mask only on tiles that need it
    // (a warp-uniform branch around the whole pass), then the row max over independent chains
    bool mods_done = false;
    if (modded && score_flags == TYLO_SCORE_SOFTCAP) {
      // Soft cap alone: if every score of the warp's rows is small against the cap (the usual case),
      // tanh is a branch-free odd polynomial on the FMA pipe for the whole tile.
      float am[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int t = 0; t < 32; t += 2)
          am[q] = max3(am[q], fabsf(__uint_as_float(sr[q][t])), fabsf(__uint_as_float(sr[q][t + 1])));
      }
      if (__all_sync(0xffffffffu, fmaxf(fmaxf(am[0], am[1]), fmaxf(am[2], am[3])) * cap_k1 < 0.4f)) {
        // cap*log2e*tanh(x), x = s*k1:  x (1 - x^2/3 + 2x^4/15 - 17x^6/315) = s * (a0 + u (a1 + u (a2 + u a3))), u = s^2
        const uint64_t a0 = pack_f32x2(cap_a0, cap_a0), a1 = pack_f32x2(cap_a1, cap_a1), a2 = pack_f32x2(cap_a2, cap_a2),
                       a3 = pack_f32x2(cap_a3, cap_a3);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            const uint64_t s2 = pack_f32x2(__uint_as_float(sr[q][t]), __uint_as_float(sr[q][t + 1]));
            const uint64_t u2 = mul_f32x2(s2, s2);
            float y0, y1;
            unpack_f32x2(mul_f32x2(s2, fma_f32x2(u2, fma_f32x2(u2, fma_f32x2(u2, a3, a2), a1), a0)), y0, y1);
            sr[q][t] = __float_as_uint(y0); sr[q][t + 1] = __float_as_uint(y1);
          }
        }
        mods_done = true;
      }
    }
    if (modded && !mods_done) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          float s = __uint_as_float(sr[q][t]) * p.scale;
          const int kv = kv0 + q * 32 + t;
          const bool cap_first = score_flags & TYLO_SCORE_SOFTCAP_FIRST;
          if ((score_flags & TYLO_SCORE_SOFTCAP) && cap_first) s = softcap(s, p.cap, inv_cap);
          if (score_flags & TYLO_SCORE_ALIBI) s = fmaf(slope, (float)(qpos - kv), s);
          if ((score_flags & TYLO_SCORE_SOFTCAP) && !cap_first) s = softcap(s, p.cap, inv_cap);
          sr[q][t] = __float_as_uint(s * kLog2e);
        }
      }
    }
    if (partial) {
      // The document-id shuffles live in their own copy of the loop: a shuffle under a per-element
      // runtime condition makes the compiler wrap every one of the 128 in a convergence barrier.
      // key kv0 + c is kept iff row_lo <= kv0 + c <= row_hi: (unsigned)(c - rel) <= row_span with
      // rel = row_lo - kv0; a row that keeps nothing gets a start no column can reach.
      const int rel = (row_any && row_doc_ok) ? row_lo - kv0 : 0x40000000;
      auto mask_pass = [&](auto with_doc) {
        constexpr bool DOCS = decltype(with_doc)::value;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            bool keep = (unsigned)(q * 32 + t - rel) <= row_span;
            if (DOCS) {
              const int key_doc = __shfl_sync(0xffffffffu, ids[q], t);   // every lane takes part, masked or not
              keep = keep && (key_doc == my_doc);
            }
            sr[q][t] = keep ? sr[q][t] : 0xff800000u;   // -inf
          }
        }
      };
      if (doc_elementwise) mask_pass(std::true_type{}); else mask_pass(std::false_type{});
    }
    float mxq[4][2];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      mxq[q][0] = -INFINITY; mxq[q][1] = -INFINITY;
#pragma unroll
      for (int t = 0; t < 32; t += 4) {
        mxq[q][0] = max3(mxq[q][0], __uint_as_float(sr[q][t]), __uint_as_float(sr[q][t + 1]));
        mxq[q][1] = max3(mxq[q][1], __uint_as_float(sr[q][t + 2]), __uint_as_float(sr[q][t + 3]));
      }
    }
    const float mx = fmaxf(fmaxf(max3(mxq[0][0], mxq[0][1], mxq[1][0]), max3(mxq[1][1], mxq[2][0], mxq[2][1])),
                           fmaxf(mxq[3][0], mxq[3][1]));
    m_true = fmaxf(m_true, mx);
    if (__all_sync(0xffffffffu, mx == -INFINITY)) {
      // every pair of this warp's 32 rows is masked in this tile (e.g. keys of another document):
      pass_empty_tile();
      continue;
    }
    // lazy rescaling: move the reference max only when it would otherwise overflow the 2^8 headroom
    const bool need = (mx > m_ref) && ((m_ref == -INFINITY) || ((mx - m_ref) * c > 8.f));
    if (__any_sync(0xffffffffu, need)) {
      if (i > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::O_READY + X), (i - 1) & 1, abort_flag, &g_attn_fwd_status, 302));
        if (!ok) break;
        tc_fence_after();
        const float f = need ? ((m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - mx) * c)) : 1.f;
        l *= f;
#pragma unroll
        for (int q = 0; q < D / 32; ++q) {
          uint32_t orr[32];
          tmem_ld32(to + q * 32, orr);
          tc_wait_ld();
#pragma unroll
          for (int t = 0; t < 32; ++t) orr[t] = __float_as_uint(__uint_as_float(orr[t]) * f);
          tmem_st32(to + q * 32, orr);
        }
        tc_wait_st();
      }
      if (need) m_ref = mx;
    }
    const float mc = (m_ref == -INFINITY) ? 0.f : m_ref * c;
    float lsq[4][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
    // Two scores per instruction on the FMA pipe: fma.rn.f32x2 for the exponent arguments and
    // add.rn.f32x2 for the running row sums (register pairs, sm_100 packed fp32).
    const uint64_t c2 = pack_f32x2(c, c), mc2 = pack_f32x2(-mc, -mc);
    uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t pk[16];
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        float x0, x1;
        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sr[q][2 * t]), __uint_as_float(sr[q][2 * t + 1])), c2, mc2), x0, x1);
        const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
        ls2[q] = add_f32x2(ls2[q], pack_f32x2(p0, p1));
        pk[t] = pack_pair<T>(p0, p1);
      }
      unpack_f32x2(ls2[q], lsq[q][0], lsq[q][1]);
      // 16 columns of packed pairs = 32 probabilities
      asm volatile(
          "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
          ::"r"(ts + q * 16), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]),
            "r"(pk[7]), "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]), "r"(pk[14]),
            "r"(pk[15]) : "memory");
    }
    l += ((lsq[0][0] + lsq[0][1]) + (lsq[1][0] + lsq[1][1])) + ((lsq[2][0] + lsq[2][1]) + (lsq[3][0] + lsq[3][1]));
    tc_wait_st();
    tc_fence_before();
    mbar_arrive(bar(SM::P_FULL + X));
  }

  // ---- epilogue: O / l, M, L   (tcgen05.ld is warp-collective: every lane loads, stores are predicated)
  float inv = 0.f;
  if (n > 0 && ok) {
    ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::O_READY + X), (n - 1) & 1, abort_flag, &g_attn_fwd_status, 303));
    tc_fence_after();
    inv = l > 0.f ? 1.f / l : 0.f;
  }
  if (ok) {
    const bool live = row < q_lim;
    T* og = O + ((size_t)(b * p.H + h) * p.Sq + (live ? row : 0)) * D;
#pragma unroll
    for (int q = 0; q < D / 32; ++q) {
      uint32_t orr[32];
      if (n > 0) { tmem_ld32(to + q * 32, orr); tc_wait_ld(); }
      uint4 out[4];
      uint32_t* ow = reinterpret_cast<uint32_t*>(out);
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const float a = (n > 0) ? __uint_as_float(orr[2 * t]) * inv : 0.f;
        const float bb = (n > 0) ? __uint_as_float(orr[2 * t + 1]) * inv : 0.f;
        ow[t] = pack_pair<T>(a, bb);
      }
      if (live) {
#pragma unroll
        for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(og + q * 32 + v * 8) = out[v];
      }
    }
    if (live) {
      const size_t si = (size_t)(b * p.H + h) * p.Sq + row;
      // m_true / m_ref are in units of c; statistics are reported in log2 units (attention!) or
      // natural units (flex)
      const float m2 = (m_true == -INFINITY) ? -INFINITY : m_true * c;
      const float lt = (m_true == -INFINITY) ? 0.f : l * fast_exp2((m_ref - m_true) * c);
      if (Mout) Mout[si] = p.natural_stats ? m2 * kLn2 : m2;
      if (Lout) Lout[si] = lt;
    }
  }
}

template <typename T, int D, uint32_t MASK, uint32_t SCORE>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, T* __restrict__ O, float* __restrict__ Mout,
                      float* __restrict__ Lout, const AttnParams p) {
  using SM = FwdSmem<D>;
  constexpr int ST = SM::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_addr(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMisc + 4);
  auto bar = [&](int i) { return sbase + SM::kBars + 8 * i; };

  const uint32_t mask_flags = (MASK == kRuntimeMods) ? p.mask_flags : MASK;
  const uint32_t score_flags = (SCORE == kRuntimeMods) ? p.score_flags : SCORE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = (p.Sq + 2 * BM - 1) / (2 * BM);
  const int qt = nqt - 1 - (int)(blockIdx.x % nqt);   // heaviest causal tiles first
  const int hb = blockIdx.x / nqt;
  const int b = hb / p.H, h = hb % p.H, hk = h / p.G;
  const int q0 = qt * 2 * BM;

  // Ragged batches (attention.jl:25-26,37-46,60): keys at or beyond k_lengths[b] are masked; 64-row
  // query blocks that start at or beyond q_lengths[b] are skipped and their output rows left untouched.
  int k_len = p.Sk, q_lim = p.Sq;
  if (p.k_lengths) { const int v = p.k_lengths[b]; k_len = v < 0 ? 0 : (v > p.Sk ? p.Sk : v); }
  if (p.q_lengths) {
    const int v = p.q_lengths[b];
    const int ql = v < 0 ? 0 : (v > p.Sq ? p.Sq : v);
    q_lim = min(p.Sq, ((ql + 63) / 64) * 64);
  }

  // key tiles each Q tile can see, as CTA-local index ranges over the union
  int t0[2], t1[2];
#pragma unroll
  for (int X = 0; X < 2; ++X) {
    const int qx = q0 + X * BM;
    t0[X] = 0; t1[X] = 0;
    if (qx < q_lim) {
      AttnParams pr = p; pr.mask_flags = mask_flags;
      int lo, hi;
      kv_range(pr, qx + p.input_pos, min(qx + BM, p.Sq) - 1 + p.input_pos, k_len, &lo, &hi);
      if (hi > lo) { t0[X] = lo / BN; t1[X] = (hi - 1) / BN + 1; }
    }
  }
  const bool actA = t1[0] > t0[0], actB = t1[1] > t0[1];
  const int jlo = actA ? (actB ? min(t0[0], t0[1]) : t0[0]) : t0[1];
  const int jhi = actA ? (actB ? max(t1[0], t1[1]) : t1[0]) : t1[1];
  const int n_tot = (actA || actB) ? jhi - jlo : 0;
  const TileRange trA = {actA ? t0[0] - jlo : 0, actA ? t1[0] - jlo : 0};
  const TileRange trB = {actB ? t0[1] - jlo : 0, actB ? t1[1] - jlo : 0};

  if (threadIdx.x == 0) {
    mbar_init(bar(SM::Q_FULL), 1); mbar_init(bar(SM::Q_FULL + 1), 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(bar(SM::K_FULL + s), 1); mbar_init(bar(SM::K_EMPTY + s), 1);
      mbar_init(bar(SM::V_FULL + s), 1); mbar_init(bar(SM::V_EMPTY + s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(SM::S_FULL + i), 1); mbar_init(bar(SM::P_FULL + i), 128); mbar_init(bar(SM::O_READY + i), 1);
    }
    mbar_init(bar(SM::DONE), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_addr(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Register split of the 384 x 168 pool: 4 x 32 x 88 + 8 x 32 x 208.  The producer and MMA-issuing
  // threads are on the latency-critical path of every hand-off: at 56 registers they spill (measured:
  // 859 TFLOP/s against 944 with 88 on the causal headline shape); the softmax rows fit in 208.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0 && n_tot > 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
#pragma unroll
        for (int X = 0; X < 2; ++X) {
          if (X == 0 ? actA : actB) {
            mbar_expect_tx(bar(SM::Q_FULL + X), SM::kTile);
#pragma unroll
            for (int cc = 0; cc < D / 64; ++cc)
              tma_load_3d(sbase + SM::kQ + X * SM::kTile + cc * (BM * 128), &tmQ, bar(SM::Q_FULL + X), cc * 64, q0 + X * BM,
                          b * p.H + h);
          }
        }
        bool ok = true;
        for (int j = 0; j < n_tot && ok; ++j) {
          const int s = j % ST;
          const int row = (jlo + j) * BN;
          if (j >= ST) ok = mbar_wait(bar(SM::K_EMPTY + s), ((j / ST) - 1) & 1, abort_flag, &g_attn_fwd_status, 101);
          if (!ok) break;
          mbar_expect_tx(bar(SM::K_FULL + s), SM::kTile);
#pragma unroll
          for (int cc = 0; cc < D / 64; ++cc)
            tma_load_3d(sbase + SM::kK + s * SM::kTile + cc * (BN * 128), &tmK, bar(SM::K_FULL + s), cc * 64, row, b * p.Hkv + hk);
          if (j >= ST) ok = mbar_wait(bar(SM::V_EMPTY + s), ((j / ST) - 1) & 1, abort_flag, &g_attn_fwd_status, 102);
          if (!ok) break;
          mbar_expect_tx(bar(SM::V_FULL + s), SM::kTile);
#pragma unroll
          for (int cc = 0; cc < D / 64; ++cc)
            tma_load_3d(sbase + SM::kV + s * SM::kTile + cc * (BN * 128), &tmV, bar(SM::V_FULL + s), cc * 64, row, b * p.Hkv + hk);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0 && n_tot > 0) {
        constexpr uint32_t idesc_qk = idesc_f16(MmaFmt<T>::v, 0, 0, BM, BN);
        constexpr uint32_t idesc_pv = idesc_f16(MmaFmt<T>::v, 0, 1, BM, D);
        auto active = [&](int X, int j) { const TileRange& t = X ? trB : trA; return j >= t.s && j < t.e; };
        // Descriptors differ only in their 14-bit start-address field: build the constant upper
        // halves once and add a pre-shifted byte offset per MMA, so that the single issuing thread
        // spends a couple of integer instructions per tcgen05.mma instead of a dependent chain.
        const uint64_t dk_hi = smem_desc_sw128(0, 16, 1024);              // K-major Q / K operands
        const uint64_t dv_hi = smem_desc_sw128(0, BN * 128, 1024);        // MN-major V operand
        auto desc_at = [](uint64_t hi, uint32_t saddr) { return hi | (uint64_t)((saddr & 0x3ffff) >> 4); };
        auto issue_qk = [&](int X, int j) {
          const uint32_t d = tmem + X * 128;
          const uint64_t qd = desc_at(dk_hi, sbase + SM::kQ + X * SM::kTile);
          const uint64_t kd = desc_at(dk_hi, sbase + SM::kK + (j % ST) * SM::kTile);
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = ((k / 4) * (BM * 128) + (k % 4) * 32) >> 4;   // compile-time constant
            mma_ss(d, qd + off, kd + off, idesc_qk, k > 0);
          }
          tc_commit(bar(SM::S_FULL + X));
        };
        auto issue_pv = [&](int X, int j) {
          const TileRange& t = X ? trB : trA;
          const uint32_t pa = tmem + X * 128;              // P: 64 columns of packed pairs
          const uint64_t vd = desc_at(dv_hi, sbase + SM::kV + (j % ST) * SM::kTile);
          const bool first = (j == t.s);
#pragma unroll
          for (int k = 0; k < BN / 16; ++k)
            mma_ts(tmem + 256 + X * 128, pa + k * 8, vd + (uint32_t)((k * 2048) >> 4), idesc_pv, !first || (k > 0));
          tc_commit(bar(SM::O_READY + X));
        };
        bool ok = true;
        if (actA) ok = ok && mbar_wait(bar(SM::Q_FULL + 0), 0, abort_flag, &g_attn_fwd_status, 201);
        if (actB) ok = ok && mbar_wait(bar(SM::Q_FULL + 1), 0, abort_flag, &g_attn_fwd_status, 201);
        ok = ok && mbar_wait(bar(SM::K_FULL + 0), 0, abort_flag, &g_attn_fwd_status, 202);
        if (ok) {
          tc_fence_after();
          if (active(0, 0)) issue_qk(0, 0);
          if (active(1, 0)) issue_qk(1, 0);
          tc_commit(bar(SM::K_EMPTY + 0));
        }
        for (int j = 0; j < n_tot && ok; ++j) {
          const int s = j % ST;
          bool v_ready = false, k_ready = false;
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            if (active(X, j)) {
              if (!v_ready) { ok = mbar_wait(bar(SM::V_FULL + s), (j / ST) & 1, abort_flag, &g_attn_fwd_status, 204); v_ready = true; }
              const TileRange& t = X ? trB : trA;
              ok = ok && mbar_wait(bar(SM::P_FULL + X), (j - t.s) & 1, abort_flag, &g_attn_fwd_status, 205);
              if (!ok) break;
              tc_fence_after();
              issue_pv(X, j);
            }
            if (j + 1 < n_tot && active(X, j + 1)) {
              if (!k_ready) {
                ok = mbar_wait(bar(SM::K_FULL + (j + 1) % ST), ((j + 1) / ST) & 1, abort_flag, &g_attn_fwd_status, 203);
                k_ready = true;
              }
              if (!ok) break;
              tc_fence_after();
              issue_qk(X, j + 1);
            }
          }
          if (!ok) break;
          tc_commit(bar(SM::V_EMPTY + s));
          if (j + 1 < n_tot) tc_commit(bar(SM::K_EMPTY + (j + 1) % ST));
        }
        // nothing may still be executing when the allocation is released
        tc_commit(bar(SM::DONE));
        mbar_drain(bar(SM::DONE), 0);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int X = (warp >= 8) ? 1 : 0;
    softmax_tile<T, D, MASK, SCORE>(p, mask_flags, score_flags, X, q0 + X * BM, jlo, X ? trB : trA, b, h, tmem, sbase,
                                    abort_flag, O, Mout, Lout, k_len, q_lim);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0 && lane == 0 && n_tot > 0) {
    // make sure none of this CTA's TMA copies is still in flight before its shared memory is released
    for (int s = 0; s < ST && s < n_tot; ++s) {
      const int last = ((n_tot - 1 - s) / ST) * ST + s;   // last tile that used stage s
      mbar_drain(bar(SM::K_FULL + s), (last / ST) & 1);
      mbar_drain(bar(SM::V_FULL + s), (last / ST) & 1);
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
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

// 3-D view (D, S, heads*batch) of a dense (D,S,H,B) array; box = 64 x 128 x 1, 128-byte swizzle.
static int32_t make_tmap(CUtensorMap* map, const void* base, int D, int S, int BH) {
  auto fn = encode_fn();
  TYLO_REQUIRE(fn, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)S * D * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)BN, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TYLO_REQUIRE(r == CUDA_SUCCESS, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TYLO_OK;
}

bool attn_fwd_sm100_supported(const AttnParams& p, int32_t dtype) {
  if (dtype != TYLO_BF16 && dtype != TYLO_F16) return false;
  if (p.Dk != p.Dv || (p.Dk != 64 && p.Dk != 128)) return false;
  if ((long long)p.Sq * p.H * p.B > 0x7fffffffLL / 2) return false;
  return true;
}

template <typename T, int D, uint32_t MASK, uint32_t SCORE>
static int32_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* O, float* M,
                          float* L, const AttnParams& p, cudaStream_t st) {
  auto kern = attn_fwd_sm100_kernel<T, D, MASK, SCORE>;
  TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::kDynamic));
  const long long grid = (long long)((p.Sq + 2 * BM - 1) / (2 * BM)) * p.H * p.B;
  kern<<<(unsigned)grid, kFwdThreads, FwdSmem<D>::kDynamic, st>>>(mq, mk, mv, (T*)O, M, L, p);
  return check_launch("attn_fwd_sm100");
}

template <typename T, int D>
static int32_t dispatch_mods(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* O, float* M,
                             float* L, const AttnParams& p, cudaStream_t st) {
  constexpr uint32_t C = TYLO_MASK_CAUSAL, W = TYLO_MASK_SLIDING, DOC = TYLO_MASK_DOCUMENT;
  const uint32_t m = p.mask_flags, s = p.score_flags;
  if (s == 0) {
    if (m == 0) return launch_fwd<T, D, 0, 0>(mq, mk, mv, O, M, L, p, st);
    if (m == C) return launch_fwd<T, D, C, 0>(mq, mk, mv, O, M, L, p, st);
    if (m == (C | W) || m == W) return launch_fwd<T, D, W, 0>(mq, mk, mv, O, M, L, p, st);
    if (m == (C | W | DOC) || m == (W | DOC)) return launch_fwd<T, D, W | DOC, 0>(mq, mk, mv, O, M, L, p, st);
  }
  if (s == TYLO_SCORE_SOFTCAP && (m == (C | W | DOC) || m == (W | DOC)))
    return launch_fwd<T, D, W | DOC, TYLO_SCORE_SOFTCAP>(mq, mk, mv, O, M, L, p, st);
  if (s == TYLO_SCORE_SOFTCAP && m == C) return launch_fwd<T, D, C, TYLO_SCORE_SOFTCAP>(mq, mk, mv, O, M, L, p, st);
  if (s == TYLO_SCORE_ALIBI && m == C) return launch_fwd<T, D, C, TYLO_SCORE_ALIBI>(mq, mk, mv, O, M, L, p, st);
  return launch_fwd<T, D, kRuntimeMods, kRuntimeMods>(mq, mk, mv, O, M, L, p, st);
}

int32_t attn_fwd_sm100(void* O, const void* Q, const void* K, const void* V, float* M, float* L, const AttnParams& p,
                       int32_t dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  if (int32_t rc = make_tmap(&mq, Q, p.Dk, p.Sq, p.H * p.B)) return rc;
  if (int32_t rc = make_tmap(&mk, K, p.Dk, p.Sk, p.Hkv * p.B)) return rc;
  if (int32_t rc = make_tmap(&mv, V, p.Dv, p.Sk, p.Hkv * p.B)) return rc;
  if (dtype == TYLO_BF16) {
    if (p.Dk == 128) return dispatch_mods<__nv_bfloat16, 128>(mq, mk, mv, O, M, L, p, st);
    return dispatch_mods<__nv_bfloat16, 64>(mq, mk, mv, O, M, L, p, st);
  }
  if (p.Dk == 128) return dispatch_mods<__half, 128>(mq, mk, mv, O, M, L, p, st);
  return dispatch_mods<__half, 64>(mq, mk, mv, O, M, L, p, st);
}


int32_t attn_fwd_sm100_status(int* out) {
  int v = 0;
  TYLO_CUDA_OK(cudaMemcpyFromSymbol(&v, g_attn_fwd_status, sizeof(int)));
  *out = v;
  if (v != 0) {
    const int zero = 0;
    TYLO_CUDA_OK(cudaMemcpyToSymbol(g_attn_fwd_status, &zero, sizeof(int)));
  }
  return TYLO_OK;
}

}  // namespace tylo
