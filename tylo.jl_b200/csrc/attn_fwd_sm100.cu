// Flash-attention forward for sm_100a: tcgen05.mma with accumulators in tensor memory, operands
// staged by TMA into a 128-byte-swizzled shared-memory ring, warp-specialised roles.
//
// One CTA owns 128 query rows of one (head, batch) and walks the 128-key tiles its mask allows.
//
//   warp 0      TMA producer: Q once, then K and V tiles through 3-stage rings (mbarrier full/empty).
//   warp 1      MMA issuer (one elected lane) and owner of the tensor-memory allocation:
//                 S[j&1] = Q K_j^T        (both operands from shared memory, 128x128xD)
//                 O     += P_j V_j        (P from tensor memory, V MN-major from shared memory)
//               S is double-buffered so that Q K_{j+1}^T runs while the softmax of tile j does.
//   warps 2..5  softmax: thread r owns query row r (= TMEM lane r).  Reads S with tcgen05.ld,
//               applies score/mask mods, keeps a running max / sum in fp32, writes P (bf16/f16)
//               back over the S columns with tcgen05.st, rescales O in TMEM only when the row
//               max grew by more than 2^8 (lazy rescaling), and writes the final O, M, L.
//
// TMEM columns: [0,128) S0/P0, [128,256) S1/P1, [256,256+D) O.   No multicast, no clusters.
// Every mbarrier wait is bounded; a time-out sets a status word and drains the CTA.
#include <cuda.h>
#include <cudaTypedefs.h>

#include "attn_dispatch.cuh"
#include "sm100_ptx.cuh"

namespace tylo {
using namespace sm100;

__device__ int g_attn_fwd_status = 0;

constexpr uint32_t kRuntimeMods = 0x80000000u;  // template value: read the flags from AttnParams
constexpr int BM = 128, BN = 128;
constexpr int kStages = 3;
constexpr int kFwdThreads = 192;

template <int D> struct FwdSmem {
  static constexpr int kTile = BM * D * 2;             // bytes of one Q / K / V tile
  static constexpr int kQ = 0;
  static constexpr int kK = kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kBars = kV + kStages * kTile;    // 8-byte mbarriers
  static constexpr int kNumBars = 1 + 4 * kStages + 2 + 2 + 1 + 1;
  static constexpr int kMisc = kBars + 8 * kNumBars;    // tmem base, abort flag
  static constexpr int kTotal = kMisc + 16;
  static constexpr int kDynamic = kTotal + 1024;        // slack for manual 1024-byte alignment
};

enum FwdBar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 1 + kStages, V_FULL = 1 + 2 * kStages, V_EMPTY = 1 + 3 * kStages,
              S_FULL = 1 + 4 * kStages, P_FULL = S_FULL + 2, O_READY = P_FULL + 2, DONE = O_READY + 1 };

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

template <typename T, int D, uint32_t MASK, uint32_t SCORE>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, T* __restrict__ O, float* __restrict__ Mout,
                      float* __restrict__ Lout, const AttnParams p) {
  using SM = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_addr(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMisc + 4);
  auto bar = [&](int i) { return sbase + SM::kBars + 8 * i; };

  const uint32_t mask_flags = (MASK == kRuntimeMods) ? p.mask_flags : MASK;
  const uint32_t score_flags = (SCORE == kRuntimeMods) ? p.score_flags : SCORE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqt = (p.Sq + BM - 1) / BM;
  const int qt = nqt - 1 - (int)(blockIdx.x % nqt);   // heaviest causal tiles first
  const int hb = blockIdx.x / nqt;
  const int b = hb / p.H, h = hb % p.H, hk = h / p.G;
  const int q0 = qt * BM;

  // key tiles this query tile can see
  int kv_lo, kv_hi;
  {
    AttnParams pr = p; pr.mask_flags = mask_flags;
    kv_range(pr, q0 + p.input_pos, min(q0 + BM, p.Sq) - 1 + p.input_pos, p.Sk, &kv_lo, &kv_hi);
  }
  const int jt0 = kv_lo / BN;
  const int n_tiles = kv_hi > kv_lo ? (kv_hi - 1) / BN - jt0 + 1 : 0;

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(K_FULL + s), 1); mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1); mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(bar(S_FULL + i), 1); mbar_init(bar(P_FULL + i), 128); }
    mbar_init(bar(O_READY), 1); mbar_init(bar(DONE), 1);
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
  const uint32_t tmem_o = tmem + 256;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
      mbar_expect_tx(bar(Q_FULL), SM::kTile);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) tma_load_3d(sbase + SM::kQ + c * (BM * 128), &tmQ, bar(Q_FULL), c * 64, q0, b * p.H + h);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        const int row = (jt0 + j) * BN;
        if (j >= kStages) ok = mbar_wait(bar(K_EMPTY + s), ((j / kStages) - 1) & 1, abort_flag, &g_attn_fwd_status, 101);
        if (!ok) break;
        mbar_expect_tx(bar(K_FULL + s), SM::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_3d(sbase + SM::kK + s * SM::kTile + c * (BN * 128), &tmK, bar(K_FULL + s), c * 64, row, b * p.Hkv + hk);
        if (j >= kStages) ok = mbar_wait(bar(V_EMPTY + s), ((j / kStages) - 1) & 1, abort_flag, &g_attn_fwd_status, 102);
        if (!ok) break;
        mbar_expect_tx(bar(V_FULL + s), SM::kTile);
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_load_3d(sbase + SM::kV + s * SM::kTile + c * (BN * 128), &tmV, bar(V_FULL + s), c * 64, row, b * p.Hkv + hk);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = idesc_f16(MmaFmt<T>::v, 0, 0, BM, BN);
      constexpr uint32_t idesc_pv = idesc_f16(MmaFmt<T>::v, 0, 1, BM, D);
      auto issue_qk = [&](int j) {
        const int s = j % kStages;
        const uint32_t d = tmem + (j & 1) * 128;
        const uint32_t qb = sbase + SM::kQ, kb = sbase + SM::kK + s * SM::kTile;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k / 4) * (BM * 128) + (k % 4) * 32;
          mma_ss(d, smem_desc_sw128(qb + off, 16, 1024), smem_desc_sw128(kb + off, 16, 1024), idesc_qk, k > 0);
        }
        tc_commit(bar(S_FULL + (j & 1)));
        tc_commit(bar(K_EMPTY + s));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, &g_attn_fwd_status, 201);
      ok = ok && mbar_wait(bar(K_FULL + 0), 0, abort_flag, &g_attn_fwd_status, 202);
      if (ok) { tc_fence_after(); issue_qk(0); }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          ok = mbar_wait(bar(K_FULL + (j + 1) % kStages), ((j + 1) / kStages) & 1, abort_flag, &g_attn_fwd_status, 203);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        const int s = j % kStages;
        ok = mbar_wait(bar(V_FULL + s), (j / kStages) & 1, abort_flag, &g_attn_fwd_status, 204);
        ok = ok && mbar_wait(bar(P_FULL + (j & 1)), (j >> 1) & 1, abort_flag, &g_attn_fwd_status, 205);
        if (!ok) break;
        tc_fence_after();
        const uint32_t pa = tmem + (j & 1) * 128;          // P: 64 columns of packed pairs
        const uint32_t vb = sbase + SM::kV + s * SM::kTile;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          mma_ts(tmem_o, pa + k * 8, smem_desc_sw128(vb + k * 2048, BN * 128, 1024), idesc_pv, (j > 0) || (k > 0));
        tc_commit(bar(V_EMPTY + s));
        tc_commit(bar(O_READY));
      }
      // nothing may still be executing when the allocation is released
      tc_commit(bar(DONE));
      mbar_drain(bar(DONE), 0);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int wq = warp & 3;                       // TMEM lane quarter this warp may touch
    const int r = wq * 32 + lane;                  // row within the tile
    const int row = q0 + r, qpos = row + p.input_pos;
    const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
    const bool modded = score_flags != 0;
    // units of the running max: raw dot products when there is no score mod (c folds the scale),
    // log2-scaled modded scores otherwise
    const float c = modded ? 1.f : p.scale * kLog2e;
    const float slope = (score_flags & TYLO_SCORE_ALIBI) ? p.slopes[h] : 0.f;
    AttnParams pr = p; pr.mask_flags = mask_flags; pr.score_flags = score_flags;
    int my_doc = 0;
    if (mask_flags & TYLO_MASK_DOCUMENT) my_doc = p.doc_q[(size_t)b * p.doc_stride + min(qpos, (int)p.Sq - 1 + p.input_pos)];

    float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int kv0 = (jt0 + j) * BN;
      int ids[4] = {0, 0, 0, 0};   // document ids of the tile's keys: lane i holds key q*32 + i
      if (mask_flags & TYLO_MASK_DOCUMENT) {
#pragma unroll
        for (int q = 0; q < 4; ++q) ids[q] = p.doc_kv[(size_t)b * p.doc_stride + min(kv0 + q * 32 + lane, p.Sk - 1)];
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + (j & 1)), (j >> 1) & 1, abort_flag, &g_attn_fwd_status, 301));
      if (!ok) break;
      tc_fence_after();
      const uint32_t ts = tmem + lane_off + (j & 1) * 128;
      uint32_t sr[4][32];
#pragma unroll
      for (int q = 0; q < 4; ++q) tmem_ld32(ts + q * 32, sr[q]);
      tc_wait_ld();

      // which elements of this tile need the element-wise mask?
      bool partial = kv0 + BN > p.Sk;
      if (mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING | TYLO_MASK_PREFIX_LM)) partial = partial || (kv0 + BN - 1 > q0 + p.input_pos);
      if (mask_flags & TYLO_MASK_SLIDING) partial = partial || (kv0 < q0 + BM - 1 + p.input_pos - p.window);
      if (mask_flags & (TYLO_MASK_DOCUMENT | TYLO_MASK_PREFIX | TYLO_MASK_PREFIX_LM)) partial = true;

      float mx = -INFINITY;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(sr[q][i]);
          const int kv = kv0 + q * 32 + i;
          if (modded) s = score_apply(pr, s * p.scale, slope, qpos, kv) * kLog2e;
          int key_doc = 0;
          if (mask_flags & TYLO_MASK_DOCUMENT) key_doc = __shfl_sync(0xffffffffu, ids[q], i);
          if (partial) {
            bool keep = kv < p.Sk;
            if (mask_flags & TYLO_MASK_CAUSAL) keep = keep && (qpos >= kv);
            if (mask_flags & TYLO_MASK_SLIDING) keep = keep && (qpos >= kv) && (qpos <= kv + p.window);
            if (mask_flags & TYLO_MASK_PREFIX) keep = keep && (kv < p.prefix_len);
            if (mask_flags & TYLO_MASK_PREFIX_LM) keep = keep && ((qpos >= kv) || (kv < p.prefix_len));
            if (mask_flags & TYLO_MASK_DOCUMENT) keep = keep && (key_doc == my_doc);
            if (!keep) s = -INFINITY;
          }
          mx = fmaxf(mx, s);
          sr[q][i] = __float_as_uint(s);
        }
      }
      m_true = fmaxf(m_true, mx);
      // lazy rescaling: move the reference max only when it would otherwise overflow the 2^8 headroom
      const bool need = (mx > m_ref) && ((m_ref == -INFINITY) || ((mx - m_ref) * c > 8.f));
      if (__any_sync(0xffffffffu, need)) {
        if (j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(O_READY), (j - 1) & 1, abort_flag, &g_attn_fwd_status, 302));
          if (!ok) break;
          tc_fence_after();
          const float f = need ? ((m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - mx) * c)) : 1.f;
          l *= f;
#pragma unroll
          for (int q = 0; q < D / 32; ++q) {
            uint32_t orr[32];
            tmem_ld32(tmem_o + lane_off + q * 32, orr);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * f);
            tmem_st32(tmem_o + lane_off + q * 32, orr);
          }
          tc_wait_st();
        }
        if (need) m_ref = mx;
      }
      const float mc = (m_ref == -INFINITY) ? 0.f : m_ref * c;
      float ls = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(sr[q][2 * i]), c, -mc));
          const float p1 = fast_exp2(fmaf(__uint_as_float(sr[q][2 * i + 1]), c, -mc));
          ls += p0 + p1;
          pk[i] = pack_pair<T>(p0, p1);
        }
        // 16 columns of packed pairs = 32 probabilities
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(ts + q * 16), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]),
              "r"(pk[7]), "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]), "r"(pk[14]),
              "r"(pk[15]) : "memory");
      }
      l += ls;
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + (j & 1)));
    }

    // ---- epilogue: O / l, M, L   (tcgen05.ld is warp-collective: every lane loads, stores are predicated)
    float inv = 0.f;
    if (n_tiles > 0 && ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(O_READY), (n_tiles - 1) & 1, abort_flag, &g_attn_fwd_status, 303));
      tc_fence_after();
      inv = l > 0.f ? 1.f / l : 0.f;
    }
    if (ok) {
      const bool live = row < p.Sq;
      T* og = O + ((size_t)(b * p.H + h) * p.Sq + (live ? row : 0)) * D;
#pragma unroll
      for (int q = 0; q < D / 32; ++q) {
        uint32_t orr[32];
        if (n_tiles > 0) { tmem_ld32(tmem_o + lane_off + q * 32, orr); tc_wait_ld(); }
        uint4 out[4];
        uint32_t* ow = reinterpret_cast<uint32_t*>(out);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float a = (n_tiles > 0) ? __uint_as_float(orr[2 * i]) * inv : 0.f;
          const float bb = (n_tiles > 0) ? __uint_as_float(orr[2 * i + 1]) * inv : 0.f;
          ow[i] = pack_pair<T>(a, bb);
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

  tc_fence_before();
  __syncthreads();
  if (warp == 0 && lane == 0 && n_tiles > 0) {
    // make sure none of this CTA's TMA copies is still in flight before its shared memory is released
    const int issued = n_tiles;
    for (int s = 0; s < kStages && s < issued; ++s) {
      const int last = ((issued - 1 - s) / kStages) * kStages + s;   // last tile that used stage s
      mbar_drain(bar(K_FULL + s), (last / kStages) & 1);
      mbar_drain(bar(V_FULL + s), (last / kStages) & 1);
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
  if (p.k_lengths || p.q_lengths) return false;   // ragged per-batch lengths: generic kernels
  if ((long long)p.Sq * p.H * p.B > 0x7fffffffLL / 2) return false;
  return true;
}

template <typename T, int D, uint32_t MASK, uint32_t SCORE>
static int32_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* O, float* M,
                          float* L, const AttnParams& p, cudaStream_t st) {
  auto kern = attn_fwd_sm100_kernel<T, D, MASK, SCORE>;
  TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::kDynamic));
  const long long grid = (long long)((p.Sq + BM - 1) / BM) * p.H * p.B;
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
