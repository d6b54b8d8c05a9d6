// Flash-attention forward for sm_100a: tcgen05.mma with accumulators in tensor memory, operands
// staged by TMA into a 128-byte-swizzled shared-memory ring, warp-specialised roles, persistent CTAs.
//
// A work item is two 128-row Q tiles A and B that share every 128-key K/V tile they visit and ping-pong on
// the tensor pipe: while the softmax warpgroup of one tile works, the MMA issuer runs the other's.  With an
// even number of query heads per KV head the two tiles are the same 128 query rows of two heads of one group
// (identical key ranges, so neither idles while the other finishes); otherwise two adjacent row blocks of one
// head.  One CTA per SM walks its share of the items: under a causal mask a slot pairs the k-th last with the
// k-th first query block of a head, so every CTA gets the same work; the next item's K, V and Q loads and its
// first Q K^T products run under the previous item's epilogue.  Launches with no more items than SMs run one
// item per CTA.
//
//   warp 0       TMA producer: per item the first K/V tile, both Q tiles, then the remaining K and V tiles
//                through rings (mbarrier full/empty).
//   warp 1       MMA issuer (one elected lane), owner of the tensor-memory allocation:
//                  S_X  = Q_X K_j^T       (both operands from shared memory, 128 x 128 x D)
//                  O_X += P_X V_j         (P from tensor memory, V MN-major from shared memory)
//   warps 2,3    work out the CTA's item table once (one item per thread), then idle: they donate their
//                registers to the softmax warpgroups.
//   warps 4..7   softmax of tile A, warps 8..11 softmax of tile B: thread r owns query row r
//                (= TMEM lane r).  Reads S with tcgen05.ld, applies score/mask mods, keeps a running
//                max / sum in fp32, writes P (bf16/f16) back over the S columns with tcgen05.st,
//                rescales O in TMEM only when the row max grew by more than 2^8 (lazy rescaling),
//                and writes the final O through shared memory with TMA stores, M and L directly.
//
//                With score mods or a non-causal mask the tile is walked 32 columns at a time in rolled
//                loops (see softmax_tile); the plain and the causal forward keep the row in registers.
//
// Element types: bf16 / f16 (kind::f16), and Float32 storage with the operands read as TF32 (kind::tf32,
// head dims 32 and 64): the tile geometry is in bytes, P stays 32-bit in place of S, and V is loaded in the
// 128-byte swizzle with 32-byte atoms, the only layout an MN-major TF32 operand may have.
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

// Slots of a softmax warp's copy of its work item in shared memory.
enum { WI_B = 0, WI_H, WI_Q0, WI_KLEN, WI_QLIM, WI_KV0, WI_N, WI_RELEASE, WI_WORDS };
// One entry of the CTA's item table in shared memory: the softmax view of tile A, of tile B, then what the
// producer and the MMA issuer need.  Filled once per CTA by the two spare warps, one item per thread, so
// that no role spends its single working thread on index arithmetic between items.
enum { IT_A = 0, IT_B = WI_WORDS, IT_NTOT = 2 * WI_WORDS, IT_JLO, IT_AS, IT_AE, IT_BS, IT_BE, IT_HK, IT_HEAD, IT_Q0, IT_BATCH,
       IT_WORDS };
constexpr int kMaxItems = 40;

// DB: bytes of one row of a Q / K / V tile (head dim x element size): 256 (16-bit D 128, TF32 D 64) or
// 128 (16-bit D 64, TF32 D 32).  A row is one or two 128-byte swizzle atoms whatever the element type, so
// the tile geometry, the TMA boxes and the descriptor arithmetic are written in bytes.
template <int DB> struct FwdSmem {
  static constexpr int kStages = (DB == 256) ? 2 : 4;
  static constexpr int kTile = BM * DB;                // bytes of one Q / K / V tile
  static constexpr int kQ = 0;                          // two Q tiles
  static constexpr int kK = 2 * kTile;
  static constexpr int kV = kK + kStages * kTile;
  static constexpr int kBars = kV + kStages * kTile;    // 8-byte mbarriers
  static constexpr int Q_FULL = 0, K_FULL = 2, K_EMPTY = K_FULL + kStages, V_FULL = K_EMPTY + kStages,
                       V_EMPTY = V_FULL + kStages, S_FULL = V_EMPTY + kStages, P_FULL = S_FULL + 2,
                       O_READY = P_FULL + 2, Q_EMPTY = O_READY + 2, O_FREE = Q_EMPTY + 1, DONE = O_FREE + 2,
                       kNumBars = DONE + 1;
  // Q_EMPTY: every Q K^T product of the finished work item has been issued, its Q tiles may be overwritten;
  // O_FREE: the softmax warpgroup has read the item's accumulator out of tensor memory.
  static constexpr int kMisc = kBars + 8 * kNumBars;    // tmem base, abort flag
  static constexpr int kItems = kMisc + 16;             // item table
  static constexpr int kStage = (kItems + kMaxItems * IT_WORDS * 4 + 1023) / 1024 * 1024;   // 8 softmax warps x 2 KB of output staging
  static constexpr int kTotal = kStage + 8 * 2048;
  static constexpr int kDynamic = kTotal + 1024;        // slack for manual 1024-byte alignment
};

template <typename T> struct MmaFmt;
template <> struct MmaFmt<__nv_bfloat16> { static constexpr int v = 1; };
template <> struct MmaFmt<__half> { static constexpr int v = 0; };
template <> struct MmaFmt<float> { static constexpr int v = 2; };    // TF32: the low 13 mantissa bits are not read

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

// Bulk tensor store of a shared-memory box (TMA), tracked in the issuing thread's bulk group.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

struct TileRange { int s, e; };  // CTA-local key-tile indices [s, e) a Q tile takes part in

// One work item: 256 query rows (tiles A and B) of one (head, batch) and the key tiles they can see.
struct FwdItem {
  int b, h, hk, q0;        // batch, query head, KV head, first query row
  int k_len, q_lim;        // ragged bounds of this batch entry
  int jlo, n_tot;          // first key tile and number of key tiles walked (union of A and B)
  TileRange tr[2];         // per Q tile, relative to jlo
};


// A CTA walks several work items.  Slot s of the launch holds one item (small launches) or the pair
// (k-th last, k-th first) query block of one head — under a causal mask the heaviest with the lightest, so
// that every slot costs about the same; CTA c takes slots c, c + gridDim.x, ...  Consecutive slots belong
// to the same head, so the CTAs running at any time share K/V tiles in L2.
// The two Q tiles of an item share every K/V tile.  With an even number of query heads per KV head they are
// the SAME 128 query rows of two heads of one group (both see the same key tiles, so neither idles while the
// other finishes); otherwise two adjacent row blocks of one head.
struct FwdPlan { int nqt, per_head, n_slots, per_slot, q_step, h_step, rows, heads; };
__device__ __forceinline__ FwdPlan fwd_plan(const AttnParams& p, int paired) {
  FwdPlan pl;
  const bool pair_heads = (p.G % 2) == 0;
  pl.rows = pair_heads ? BM : 2 * BM;
  pl.heads = pair_heads ? 2 : 1;
  pl.q_step = pair_heads ? 0 : BM;
  pl.h_step = pair_heads ? 1 : 0;
  pl.nqt = (p.Sq + pl.rows - 1) / pl.rows;
  pl.per_slot = paired == 2 ? 2 : 1;      // 2: a slot holds a (heavy, light) pair of query blocks
  pl.per_head = paired == 2 ? (pl.nqt + 1) / 2 : pl.nqt;
  pl.n_slots = pl.per_head * (p.H / pl.heads) * p.B;
  return pl;
}
// Query block of entry e of slot s, or -1 if the slot has no such entry (middle block of an odd count).
__device__ __forceinline__ int fwd_slot_block(const FwdPlan& pl, int s, int e, int& hb) {
  hb = s / pl.per_head;
  const int k = s % pl.per_head;
  const int heavy = pl.nqt - 1 - k;
  if (e == 0) return heavy;
  return (k == heavy) ? -1 : k;
}

// bm_t0 / bm_t1: with a host-built block list, the key tiles [t0, t1) that hold every listed block of the rows of
// Q tile A and B (worked out by a whole warp, see the kernel); unused otherwise.
__device__ __forceinline__ FwdItem fwd_item(const AttnParams& p, const FwdPlan& pl, uint32_t mask_flags, int hb, int qt,
                                            const int* bm_t0 = nullptr, const int* bm_t1 = nullptr) {
  FwdItem it;
  const int hpb = p.H / pl.heads;
  it.b = hb / hpb; it.h = (hb % hpb) * pl.heads; it.hk = it.h / p.G; it.q0 = qt * pl.rows;
  // Ragged batches (attention.jl:25-26,37-46,60): keys at or beyond k_lengths[b] are masked; 64-row
  // query blocks that start at or beyond q_lengths[b] are skipped and their output rows left untouched.
  it.k_len = p.Sk; it.q_lim = p.Sq;
  if (p.k_lengths) { const int v = p.k_lengths[it.b]; it.k_len = v < 0 ? 0 : (v > p.Sk ? p.Sk : v); }
  if (p.q_lengths) {
    const int v = p.q_lengths[it.b];
    const int ql = v < 0 ? 0 : (v > p.Sq ? p.Sq : v);
    it.q_lim = min(p.Sq, ((ql + 63) / 64) * 64);
  }
  // key tiles each Q tile can see, as item-local index ranges over the union
  int t0[2], t1[2];
#pragma unroll
  for (int X = 0; X < 2; ++X) {
    const int qx = it.q0 + X * pl.q_step;
    t0[X] = 0; t1[X] = 0;
    if (qx < it.q_lim && p.bm_count) {
      // flex.jl:107-182: the list replaces the analytic range (the mask mod still runs per pair, below)
      t0[X] = bm_t0[X]; t1[X] = min(bm_t1[X], (it.k_len + BN - 1) / BN);
      if (t1[X] <= t0[X]) { t0[X] = 0; t1[X] = 0; }
    } else if (qx < it.q_lim) {
      AttnParams pr = p; pr.mask_flags = mask_flags;
      int lo, hi;
      kv_range(pr, qx + p.input_pos, min(qx + BM, p.Sq) - 1 + p.input_pos, it.k_len, &lo, &hi);
      if (hi > lo) { t0[X] = lo / BN; t1[X] = (hi - 1) / BN + 1; }
    }
  }
  const bool actA = t1[0] > t0[0], actB = t1[1] > t0[1];
  it.jlo = actA ? (actB ? min(t0[0], t0[1]) : t0[0]) : t0[1];
  const int jhi = actA ? (actB ? max(t1[0], t1[1]) : t1[0]) : t1[1];
  it.n_tot = (actA || actB) ? jhi - it.jlo : 0;
  it.tr[0] = {actA ? t0[0] - it.jlo : 0, actA ? t1[0] - it.jlo : 0};
  it.tr[1] = {actB ? t0[1] - it.jlo : 0, actB ? t1[1] - it.jlo : 0};
  return it;
}

// Rare path of the lazy rescaling, kept out of line so that its registers do not weigh on the tile loop:
// multiplies this thread's accumulator row (COLS fp32 columns of tensor memory) by f.
template <int COLS>
__device__ __noinline__ void scale_accumulator_row(uint32_t to, float f) {
#pragma unroll 1
  for (int q = 0; q < COLS / 8; ++q) {
    uint32_t v[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(to + q * 8) : "memory");
    tc_wait_ld();
#pragma unroll
    for (int t = 0; t < 8; ++t) v[t] = __float_as_uint(__uint_as_float(v[t]) * f);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(to + q * 8), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
  }
  tc_wait_st();
}

// Softmax / epilogue of one Q tile of one work item (one warpgroup, 128 threads).  Returns false when a
// bounded wait gave up.
template <typename T, int D, uint32_t MASK, uint32_t SCORE>
__device__ __forceinline__ bool softmax_tile(const AttnParams& p, const uint32_t mask_flags,
                                             const uint32_t score_flags, const int X, volatile const int* wi,
                                             const uint32_t tmem, const uint32_t sbase, volatile int* abort_flag,
                                             const CUtensorMap* tmO, float* __restrict__ Mout, float* __restrict__ Lout,
                                             const int ph0, const bool single_item) {
  // wi: this warp's copy of the work item in shared memory (see WI_*), read where a value is used instead
  // of being carried in registers through the tile loop, whose 128 scores per thread leave no room;
  // ph0: key tiles this warpgroup has walked in the CTA's earlier work items (mbarrier phases go on
  // counting across items).
  using SM = FwdSmem<D * (int)sizeof(T)>;
  // Two forms of the tile loop.  Register-resident (no mods, at most a causal mask): the row's 128 scores
  // stay in registers from the load to the probabilities.  Chunked (everything else): mods, mask and max run
  // over 32 columns at a time in a rolled loop, the changed scores go back to tensor memory and a second
  // rolled loop turns them into probabilities; the loop body is a quarter of the unrolled tile, which matters
  // because the mod and mask code of a whole unrolled tile does not fit the instruction cache next to the other
  // roles (config-4 mods: 0.336 ms register-resident, 0.279 ms chunked; the plain causal forward is 7 % slower
  // chunked, since it reads every score twice for nothing).
  constexpr bool kChunked = (MASK & ~(uint32_t)TYLO_MASK_CAUSAL) != 0 || SCORE != 0;
  auto bar = [&](int i) { return sbase + SM::kBars + 8 * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wq = warp & 3;                       // TMEM lane quarter this warp may touch
  const int r = wq * 32 + lane;                  // row within the tile
  const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
  const uint32_t ts = tmem + lane_off + X * 128;
  const uint32_t to = tmem + lane_off + 256 + X * 128;
  const bool modded = score_flags != 0;
  // units of the running max: raw dot products when there is no score mod (c folds the scale),
  // log2-scaled modded scores otherwise
  const float c = modded ? 1.f : p.scale * kLog2e;
  const float slope = (score_flags & TYLO_SCORE_ALIBI) ? p.slopes[wi[WI_H]] : 0.f;
  const float inv_cap = 1.f / p.cap;
  int my_doc = 0;
  if (mask_flags & TYLO_MASK_DOCUMENT)
    my_doc = p.doc_q[(size_t)wi[WI_B] * p.doc_stride + min(wi[WI_Q0] + r + p.input_pos, (int)p.Sq - 1 + p.input_pos)];
  const int n = wi[WI_N];

  // soft cap as s * P(s^2) with the constants of the tanh series folded in (see below)
  const float cap_k1 = p.scale * inv_cap;
  const float cap_a0 = cap_k1 * p.cap * kLog2e, cap_u = cap_k1 * cap_k1;
  const float cap_a1 = -0.33333334f * cap_a0 * cap_u, cap_a2 = 0.13333334f * cap_a0 * cap_u * cap_u,
              cap_a3 = -0.05396825f * cap_a0 * cap_u * cap_u * cap_u;

  float m_ref = -INFINITY, m_true = -INFINITY, l = 0.f;
  bool ok = true;
  for (int i = 0; i < n && ok; ++i) {
    // (read before the wait for S: none of it depends on the scores)
    const int kv0 = wi[WI_KV0] + i * BN;
    const int q_lo = wi[WI_Q0] + p.input_pos, q_hi = q_lo + BM - 1;
    const int k_len_i = wi[WI_KLEN];
    int ids[4] = {0, 0, 0, 0};   // document ids of the tile's keys: lane t holds key q*32 + t
    bool doc_uniform = false;
    if (mask_flags & TYLO_MASK_DOCUMENT) {
#pragma unroll
      for (int q = 0; q < 4; ++q) ids[q] = p.doc_kv[(size_t)wi[WI_B] * p.doc_stride + min(kv0 + q * 32 + lane, p.Sk - 1)];
      const int id0 = __shfl_sync(0xffffffffu, ids[0], 0);
      doc_uniform = __all_sync(0xffffffffu, ids[0] == id0 && ids[1] == id0 && ids[2] == id0 && ids[3] == id0);
    }
    // BiasScore (mods.jl:219-237): this row's 32 table entries for chunk q, local row index, heads and batch
    // broadcast by modulo; 16-byte loads when the row start is aligned, guarded scalars otherwise.  Asked for a
    // chunk ahead of their use (the first chunk before the scores are even there), so that the latency of the
    // table is not in the tile's chain.
    const bool has_bias = MASK == kRuntimeMods && (score_flags & TYLO_SCORE_BIAS);
    auto load_bias = [&](float (&bias_row)[32], const int q) {
      if (!has_bias) return;
      const int kvq = kv0 + q * 32;
      const float* bp = p.bias + bias_index(p, wi[WI_B], wi[WI_H], min(wi[WI_Q0] + r, p.Sq - 1), 0);
      if ((p.Sk & 3) == 0 && kvq + 32 <= p.Sk) {
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(bp + kvq + t));
          bias_row[t] = f.x; bias_row[t + 1] = f.y; bias_row[t + 2] = f.z; bias_row[t + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int t = 0; t < 32; ++t) bias_row[t] = (kvq + t < p.Sk) ? __ldg(bp + kvq + t) : 0.f;
      }
    };
    float bias_a[32], bias_b[32];      // two chunks of table entries in flight (bias tables only)
    load_bias(bias_a, 0);
    // Host-built block list (mods.jl:436-476, walk of flex.jl:107-182): state of the (query block, key block) that
    // each 32-column chunk of this warp's 32 rows lies in, two bits per chunk: 0 not listed (its pairs contribute
    // nothing), 1 listed (the mask mod decides per pair), 2 listed and marked full (only the key-length bound).
    // Block edges are multiples of 32, so a warp's rows and a chunk's keys never straddle a block.  32 list
    // entries per step; the ids of one query block are distinct.
    const bool listed_walk = MASK == kRuntimeMods && p.bm_count != nullptr;
    int bst = 0;
    if (listed_walk) {
      const int qb = min(wi[WI_Q0] + wq * 32, p.Sq - 1) / p.bm_tm;
      const int nb = min(p.bm_count[qb], p.bm_stride);
      for (int base = 0; base < nb; base += 32) {
        const int t = base + lane;
        const int j = t < nb ? p.bm_idx[(size_t)qb * p.bm_stride + t] : -1;
        const bool f = t < nb && p.bm_full[(size_t)qb * p.bm_stride + t] != 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const bool hit = j == (kv0 + q * 32) / p.bm_tn;
          if (__any_sync(0xffffffffu, hit)) bst |= (__any_sync(0xffffffffu, hit && f) ? 2 : 1) << (2 * q);
        }
      }
    }
    ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::S_FULL + X), (ph0 + i) & 1, abort_flag, &g_attn_fwd_status, 301));
    if (!ok) break;
    tc_fence_after();
    // P = 0 for the whole tile: nothing to load, exponentiate or rescale
    auto pass_empty_tile = [&]() {
      uint32_t z[32];
#pragma unroll
      for (int t = 0; t < 32; ++t) z[t] = 0u;
#pragma unroll
      for (int cq = 0; cq < (sizeof(T) == 4 ? 4 : 2); ++cq) tmem_st32(ts + cq * 32, z);   // 128 packed pairs or 128 fp32
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(SM::P_FULL + X));
    };
    if (!listed_walk && (mask_flags & TYLO_MASK_DOCUMENT) && doc_uniform && __all_sync(0xffffffffu, ids[0] != my_doc)) {
      // all 128 keys belong to one document that none of this warp's 32 rows belongs to
      pass_empty_tile();
      continue;
    }
    if (listed_walk && bst == 0) {
      // none of the tile's key blocks is listed for this warp's query block
      pass_empty_tile();
      continue;
    }
    // which tiles need the element-wise mask?
    bool partial = kv0 + BN > k_len_i;
    if (mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING | TYLO_MASK_PREFIX_LM)) partial = partial || (kv0 + BN - 1 > q_lo);
    if (mask_flags & TYLO_MASK_SLIDING) partial = partial || (kv0 < q_hi - p.window);
    if (mask_flags & (TYLO_MASK_PREFIX | TYLO_MASK_PREFIX_LM)) partial = true;
    if (MASK == kRuntimeMods && p.n_or > 0) partial = true;
    if (listed_walk) partial = true;
    if (mask_flags & TYLO_MASK_DOCUMENT) partial = partial || !doc_uniform || __any_sync(0xffffffffu, ids[0] != my_doc);
    const bool doc_elementwise = (mask_flags & TYLO_MASK_DOCUMENT) && !doc_uniform;
    const bool row_doc_ok = !(mask_flags & TYLO_MASK_DOCUMENT) || doc_elementwise || (__shfl_sync(0xffffffffu, ids[0], 0) == my_doc);

    // Every mask term except an element-wise document comparison keeps ONE interval of keys per row:
    // [row_lo, row_hi] (mods.jl:101-167 reduced to bounds).  Inside a tile the test is then one unsigned
    // compare per element against the tile-relative start: key kv0 + c is kept iff row_lo <= kv0 + c <= row_hi,
    // (unsigned)(c - rel) <= span with rel = row_lo - kv0; a row that keeps nothing gets a start no column
    // can reach.  OrMask in disjunctive normal form (mods.jl:164-167): every conjunction of affine terms is
    // one more interval, a key is kept if any of them holds it (document terms inside an OR run on the
    // fp32-arithmetic kernels, see the dispatch).
    int rels[1 + kMaxOrClauses]; unsigned spans[1 + kMaxOrClauses];
    rels[0] = 0x40000000; spans[0] = 0u;
    if (partial) {
      const int qpos = wi[WI_Q0] + r + p.input_pos;
      int row_lo = 0, row_hi = wi[WI_KLEN] - 1;
      if (mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) row_hi = min(row_hi, qpos);
      if (mask_flags & TYLO_MASK_SLIDING) row_lo = max(row_lo, qpos - p.window);
      if (mask_flags & TYLO_MASK_PREFIX) row_hi = min(row_hi, p.prefix_len - 1);
      if (mask_flags & TYLO_MASK_PREFIX_LM) row_hi = min(row_hi, max(qpos, p.prefix_len - 1));
      const bool row_any = row_hi >= row_lo;
      spans[0] = row_any ? (unsigned)(row_hi - row_lo) : 0u;
      rels[0] = (row_any && row_doc_ok) ? row_lo - kv0 : 0x40000000;
      if (MASK == kRuntimeMods && p.n_or > 0) {
#pragma unroll
        for (int ci = 0; ci < kMaxOrClauses; ++ci) {
          rels[1 + ci] = 0x40000000; spans[1 + ci] = 0u;
          if (ci < p.n_or) {
            const MaskClause& cl = p.or_clause[ci];
            int lo = 0, hi = wi[WI_KLEN] - 1;
            if (cl.flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) hi = min(hi, qpos);
            if (cl.flags & TYLO_MASK_SLIDING) lo = max(lo, qpos - cl.window);
            if (cl.flags & TYLO_MASK_PREFIX) hi = min(hi, cl.prefix_len - 1);
            if (cl.flags & TYLO_MASK_PREFIX_LM) hi = min(hi, max(qpos, cl.prefix_len - 1));
            if (hi >= lo) { rels[1 + ci] = lo - kv0; spans[1 + ci] = (unsigned)(hi - lo); }
          }
        }
      }
    }

    // ---- the steps of one chunk: 32 key columns (chunk q of the tile) of this thread's row ----
    // score mods (compile-time selected)
    auto apply_mods = [&](uint32_t (&v)[32], const int q, const float (&bias_row)[32]) {
      if (score_flags == TYLO_SCORE_SOFTCAP) {
        // Soft cap alone: if every score of the warp's rows is small against the cap (the usual case),
        // tanh is a branch-free odd polynomial on the FMA pipe for the whole chunk.
        float am0 = 0.f, am1 = 0.f;
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          am0 = max3(am0, fabsf(__uint_as_float(v[t])), fabsf(__uint_as_float(v[t + 1])));
          am1 = max3(am1, fabsf(__uint_as_float(v[t + 2])), fabsf(__uint_as_float(v[t + 3])));
        }
        if (__all_sync(0xffffffffu, fmaxf(am0, am1) * cap_k1 < 0.4f)) {
          // cap*log2e*tanh(x), x = s*k1:  x (1 - x^2/3 + 2x^4/15 - 17x^6/315) = s * (a0 + u (a1 + u (a2 + u a3))), u = s^2
          const uint64_t a0 = pack_f32x2(cap_a0, cap_a0), a1 = pack_f32x2(cap_a1, cap_a1), a2 = pack_f32x2(cap_a2, cap_a2),
                         a3 = pack_f32x2(cap_a3, cap_a3);
#pragma unroll
          for (int t = 0; t < 32; t += 2) {
            const uint64_t s2 = pack_f32x2(__uint_as_float(v[t]), __uint_as_float(v[t + 1]));
            const uint64_t u2 = mul_f32x2(s2, s2);
            float y0, y1;
            unpack_f32x2(mul_f32x2(s2, fma_f32x2(u2, fma_f32x2(u2, fma_f32x2(u2, a3, a2), a1), a0)), y0, y1);
            v[t] = __float_as_uint(y0); v[t + 1] = __float_as_uint(y1);
          }
          return;
        }
      }
      const int kvq = kv0 + q * 32;
      const int qpos = wi[WI_Q0] + r + p.input_pos;
      if (!(score_flags & TYLO_SCORE_SOFTCAP)) {
        // Additive mods only (ALiBi, bias tables): one fused multiply-add per element and mod, in log2 units, no
        // per-element tests of flags that are only known at run time, no integer-to-float conversion (the
        // position difference of column t is that of column 0 minus t).
        const float k2 = p.scale * kLog2e;
        if (score_flags & TYLO_SCORE_ALIBI) {
          const float sl2 = slope * kLog2e, d0 = (float)(qpos - kvq);
          const bool bias_too = MASK == kRuntimeMods && (score_flags & TYLO_SCORE_BIAS);
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const float add = fmaf(sl2, d0 - (float)t, bias_too ? bias_row[t] * kLog2e : 0.f);
            v[t] = __float_as_uint(fmaf(__uint_as_float(v[t]), k2, add));
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = __float_as_uint(fmaf(__uint_as_float(v[t]), k2, bias_row[t] * kLog2e));
        }
        return;
      }
      const bool cap_first = score_flags & TYLO_SCORE_SOFTCAP_FIRST;
#pragma unroll
      for (int t = 0; t < 32; ++t) {
        float s = __uint_as_float(v[t]) * p.scale;
        if ((score_flags & TYLO_SCORE_SOFTCAP) && cap_first) s = softcap(s, p.cap, inv_cap);
        if (score_flags & TYLO_SCORE_ALIBI) s = fmaf(slope, (float)(qpos - (kvq + t)), s);
        if (MASK == kRuntimeMods && (score_flags & TYLO_SCORE_BIAS)) s += bias_row[t];
        if ((score_flags & TYLO_SCORE_SOFTCAP) && !cap_first) s = softcap(s, p.cap, inv_cap);
        v[t] = __float_as_uint(s * kLog2e);
      }
    };
    // element-wise mask (only on tiles that need it: a warp-uniform branch around the whole pass)
    auto apply_mask = [&](uint32_t (&v)[32], const int q) {
      const int sh = q * 32;
      if (listed_walk) {
        const int st = (bst >> (2 * q)) & 3;
        if (st != 1) {
          // not listed: nothing is kept; marked full: the mask mod is skipped, keys below the length are kept
          const int lim = st == 2 ? k_len_i - kv0 - sh : 0;
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = (t < lim) ? v[t] : 0xff800000u;
          return;
        }
      }
      if (MASK == kRuntimeMods && p.n_or > 0) {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          bool keep = false;
#pragma unroll
          for (int ci = 0; ci < 1 + kMaxOrClauses; ++ci) keep = keep || ((unsigned)(sh + t - rels[ci]) <= spans[ci]);
          v[t] = keep ? v[t] : 0xff800000u;   // -inf
        }
      } else if (doc_elementwise) {
        // The document-id shuffles live in their own copy of the loop: a shuffle under a per-element
        // runtime condition makes the compiler wrap every one of them in a convergence barrier.
        const int idq = q == 0 ? ids[0] : (q == 1 ? ids[1] : (q == 2 ? ids[2] : ids[3]));
        const int relq = rels[0] - sh;
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          const int key_doc = __shfl_sync(0xffffffffu, idq, t);   // every lane takes part, masked or not
          v[t] = ((unsigned)(t - relq) <= spans[0] && key_doc == my_doc) ? v[t] : 0xff800000u;
        }
      } else {
        const int relq = rels[0] - sh;
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = ((unsigned)(t - relq) <= spans[0]) ? v[t] : 0xff800000u;
      }
    };
    // row max over two independent chains
    auto chunk_max = [&](const uint32_t (&v)[32]) -> float {
      float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
      for (int t = 0; t < 32; t += 4) {
        m0 = max3(m0, __uint_as_float(v[t]), __uint_as_float(v[t + 1]));
        m1 = max3(m1, __uint_as_float(v[t + 2]), __uint_as_float(v[t + 3]));
      }
      return fmaxf(m0, m1);
    };

    float mx;
    uint32_t sr[4][32];     // the whole tile's scores of this row (register-resident form only)
    if constexpr (!kChunked) {
#pragma unroll
      for (int q = 0; q < 4; ++q) tmem_ld32(ts + q * 32, sr[q]);
      tc_wait_ld();
      if (modded) {
#pragma unroll
        for (int q = 0; q < 4; ++q) apply_mods(sr[q], q, bias_a);      // (never a bias table in this form)
      }
      if (partial) {
#pragma unroll
        for (int q = 0; q < 4; ++q) apply_mask(sr[q], q);
      }
      mx = fmaxf(fmaxf(chunk_max(sr[0]), chunk_max(sr[1])), fmaxf(chunk_max(sr[2]), chunk_max(sr[3])));
    } else {
      // Pass 1 of the chunked form: mods, mask and max chunk by chunk, the changed scores written back to
      // tensor memory; the next chunk's load is in flight while the current one is worked on.
      uint32_t a[32], b[32];
      float mxa = -INFINITY, mxb = -INFINITY;
      const bool changed = modded || partial;
      tmem_ld32(ts, a);
      tc_wait_ld_for(a);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int qa = 2 * h, qb = 2 * h + 1;
        tmem_ld32(ts + qb * 32, b);
        load_bias(bias_b, qb);
        if (modded) apply_mods(a, qa, bias_a);
        if (partial) apply_mask(a, qa);
        mxa = fmaxf(mxa, chunk_max(a));
        if (changed) tmem_st32(ts + qa * 32, a);
        tc_wait_ld_for(b);
        if (h == 0) { tmem_ld32(ts + 64, a); load_bias(bias_a, 2); }
        if (modded) apply_mods(b, qb, bias_b);
        if (partial) apply_mask(b, qb);
        mxb = fmaxf(mxb, chunk_max(b));
        if (changed) tmem_st32(ts + qb * 32, b);
        if (h == 0) tc_wait_ld_for(a);
      }
      mx = fmaxf(mxa, mxb);
      if (changed) tc_wait_st();      // pass 2 reads them back
    }
    m_true = fmaxf(m_true, mx);
    if (__all_sync(0xffffffffu, mx == -INFINITY)) {
      // every pair of this warp's 32 rows is masked in this tile (e.g. keys of another document):
      pass_empty_tile();
      continue;
    }
    // lazy rescaling: move the reference max only when it would otherwise overflow the 2^8 headroom.
    // A row that has not met an unmasked key yet (m_ref = -inf) has l = 0 and a zero accumulator row: its
    // reference moves for free.  Only rows that have accumulated something need O and l scaled, which
    // waits for this tile's previous P V product; that is rare and kept out of line.
    const bool need = (mx > m_ref) && ((m_ref == -INFINITY) || ((mx - m_ref) * c > 8.f));
    const bool scale = need && (m_ref != -INFINITY);
    if (__any_sync(0xffffffffu, scale)) {
      if (i > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::O_READY + X), (ph0 + i - 1) & 1, abort_flag, &g_attn_fwd_status, 302));
        if (!ok) break;
        tc_fence_after();
        const float f = scale ? fast_exp2((m_ref - mx) * c) : 1.f;
        l *= f;
        scale_accumulator_row<D>(to, f);
      }
    }
    if (need) m_ref = mx;
    const float mc = (m_ref == -INFINITY) ? 0.f : m_ref * c;
    // Two scores per instruction on the FMA pipe: fma.rn.f32x2 for the exponent arguments and
    // add.rn.f32x2 for the running row sums (register pairs, sm_100 packed fp32).
    const uint64_t c2 = pack_f32x2(c, c), mc2 = pack_f32x2(-mc, -mc);
    // P of one chunk: 32 probabilities as 16 columns of packed pairs; returns their sum
    auto exp_chunk = [&](const uint32_t (&v)[32], const int q) -> float {
      uint64_t ls2 = 0ull;
      auto st16 = [&](uint32_t col, const uint32_t (&pk)[16]) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
            ::"r"(col), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]),
              "r"(pk[7]), "r"(pk[8]), "r"(pk[9]), "r"(pk[10]), "r"(pk[11]), "r"(pk[12]), "r"(pk[13]), "r"(pk[14]),
              "r"(pk[15]) : "memory");
      };
      if constexpr (sizeof(T) == 4) {
        // TF32 operand: the probabilities stay 32-bit, in place of their scores, 16 columns per store
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t pk[16];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[hh * 16 + 2 * t]), __uint_as_float(v[hh * 16 + 2 * t + 1])), c2, mc2),
                         x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            ls2 = add_f32x2(ls2, pack_f32x2(p0, p1));
            pk[2 * t] = __float_as_uint(p0); pk[2 * t + 1] = __float_as_uint(p1);
          }
          st16(ts + q * 32 + hh * 16, pk);
        }
      } else {
        uint32_t pk[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[2 * t]), __uint_as_float(v[2 * t + 1])), c2, mc2), x0, x1);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          ls2 = add_f32x2(ls2, pack_f32x2(p0, p1));
          pk[t] = pack_pair<T>(p0, p1);
        }
        st16(ts + q * 16, pk);      // 16 columns of packed pairs = 32 probabilities
      }
      float s0, s1;
      unpack_f32x2(ls2, s0, s1);
      return s0 + s1;
    };
    if constexpr (!kChunked) {
      const float s0 = exp_chunk(sr[0], 0), s1 = exp_chunk(sr[1], 1), s2 = exp_chunk(sr[2], 2), s3 = exp_chunk(sr[3], 3);
      l += (s0 + s1) + (s2 + s3);
    } else {
      // Pass 2: P chunk q lands on the columns of score chunk q / 2, which has been read by then.
      uint32_t a[32], b[32];
      float lt = 0.f;
      tmem_ld32(ts, a);
      tc_wait_ld_for(a);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int qa = 2 * h, qb = 2 * h + 1;
        tmem_ld32(ts + qb * 32, b);
        const float sa = exp_chunk(a, qa);
        tc_wait_ld_for(b);
        if (h == 0) tmem_ld32(ts + 64, a);
        const float sb = exp_chunk(b, qb);
        if (h == 0) tc_wait_ld_for(a);
        lt += sa + sb;
      }
      l += lt;
    }
    tc_wait_st();
    tc_fence_before();
    mbar_arrive(bar(SM::P_FULL + X));
  }

  // ---- epilogue: O / l, M, L   (tcgen05.ld is warp-collective: every lane loads, stores are predicated)
  float inv = 0.f;
  if (n > 0 && ok) {
    ok = __all_sync(0xffffffffu, mbar_wait(bar(SM::O_READY + X), (ph0 + n - 1) & 1, abort_flag, &g_attn_fwd_status, 303));
    tc_fence_after();
    inv = l > 0.f ? 1.f / l : 0.f;
  }
  if (ok) {
    const int row = wi[WI_Q0] + r;
    const bool live = row < wi[WI_QLIM];
    // The whole accumulator row is read out and packed first, so that the MMA issuer can start the next
    // work item's P V products while this warpgroup stores.
    // A box is 32 rows x 64 bytes: 32 columns of a 16-bit type, 16 columns of fp32.
    constexpr int kBoxes = D * (int)sizeof(T) / 64, kBoxCols = 64 / (int)sizeof(T);
    uint4 out[kBoxes][4];
#pragma unroll
    for (int q = 0; q < D / 32; ++q) {
      uint32_t orr[32];
      if (n > 0) { tmem_ld32(to + q * 32, orr); tc_wait_ld(); }
      if constexpr (sizeof(T) == 4) {
        uint32_t* ow = reinterpret_cast<uint32_t*>(out[2 * q]);     // two boxes per 32 accumulator columns
#pragma unroll
        for (int t = 0; t < 32; ++t) ow[t] = (n > 0) ? __float_as_uint(__uint_as_float(orr[t]) * inv) : 0u;
      } else {
        uint32_t* ow = reinterpret_cast<uint32_t*>(out[q]);
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          const float a = (n > 0) ? __uint_as_float(orr[2 * t]) * inv : 0.f;
          const float bb = (n > 0) ? __uint_as_float(orr[2 * t + 1]) * inv : 0.f;
          ow[t] = pack_pair<T>(a, bb);
        }
      }
    }
    if (wi[WI_RELEASE]) {
      tc_fence_before();
      mbar_arrive(bar(SM::O_FREE + X));
    }
    // Output rows leave through shared memory: each warp stages boxes of 32 rows x 64 bytes (2 KB, 64-byte swizzle,
    // conflict-free 16-byte stores) and one lane hands the box to the TMA unit, which writes whole sectors
    // and clips rows beyond Sq.  Row-by-row 16-byte stores straight from the registers would touch 32
    // lines per instruction and hold up every other shared- and global-memory instruction of the SM.
    // (q_lim is a multiple of 64 and a warp's first row of 32: a warp's rows are all live or all not.)
    // A CTA with a single work item has nothing to hide the stores under, but its Q tile is free by now
    // (the accumulator being complete means every Q K^T product has run; n > 0 means the tile was awaited):
    // the warp's boxes go into its quarter of that tile, one buffer each, and no box waits for the one before.
    if (__shfl_sync(0xffffffffu, (int)live, 0)) {
      const bool wide = single_item && n > 0;
      const uint32_t buf0 = wide ? sbase + SM::kQ + X * SM::kTile + wq * (SM::kTile / 4) : sbase + SM::kStage + (warp - 4) * 2048;
      const int row0 = wi[WI_Q0] + wq * 32, bh = wi[WI_B] * p.H + wi[WI_H];
      auto stage = [&](int q, uint32_t buf) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint32_t dst = buf + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(out[q][v].x), "r"(out[q][v].y),
                       "r"(out[q][v].z), "r"(out[q][v].w) : "memory");
        }
      };
      if (wide) {
#pragma unroll
        for (int q = 0; q < kBoxes; ++q) stage(q, buf0 + q * 2048);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int q = 0; q < kBoxes; ++q) tma_store_3d(tmO, buf0 + q * 2048, q * kBoxCols, row0, bh);
          bulk_commit();
        }
      } else {
#pragma unroll
        for (int q = 0; q < kBoxes; ++q) {
          if (lane == 0) bulk_wait_read();          // the box before this one has been read out of the buffer
          __syncwarp();
          stage(q, buf0);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) { tma_store_3d(tmO, buf0, q * kBoxCols, row0, bh); bulk_commit(); }
        }
      }
    }
    if (live) {
      const size_t si = (size_t)(wi[WI_B] * p.H + wi[WI_H]) * p.Sq + row;
      // m_true / m_ref are in units of c; statistics are reported in log2 units (attention!) or
      // natural units (flex)
      const float m2 = (m_true == -INFINITY) ? -INFINITY : m_true * c;
      const float lt = (m_true == -INFINITY) ? 0.f : l * fast_exp2((m_ref - m_true) * c);
      if (Mout) Mout[si] = p.natural_stats ? m2 * kLn2 : m2;
      if (Lout) Lout[si] = lt;
    }
  }
  return ok;
}

template <typename T, int D, uint32_t MASK, uint32_t SCORE>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                      float* __restrict__ Mout,
                      float* __restrict__ Lout, const AttnParams p, const int paired) {
  using SM = FwdSmem<D * (int)sizeof(T)>;
  constexpr int ST = SM::kStages;
  constexpr int DB = D * (int)sizeof(T);          // bytes of a tile row
  constexpr int kAtom = 128 / (int)sizeof(T);      // elements of one 128-byte swizzle atom (one TMA box)
  constexpr bool kTf32 = sizeof(T) == 4;           // fp32 storage, operands read as TF32
  constexpr int kKeysPerMma = 32 / (int)sizeof(T); // K extent of one tcgen05.mma: 32 bytes
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_addr(smem);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kMisc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kMisc + 4);
  auto bar = [&](int i) { return sbase + SM::kBars + 8 * i; };

  const uint32_t mask_flags = (MASK == kRuntimeMods) ? p.mask_flags : MASK;
  const uint32_t score_flags = (SCORE == kRuntimeMods) ? p.score_flags : SCORE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const FwdPlan plan = fwd_plan(p, paired);
  // items of this CTA: entries e of the slots blockIdx.x, blockIdx.x + gridDim.x, ... (the launch keeps the
  // count within the table)
  const int n_local = min(kMaxItems, (plan.n_slots - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x * plan.per_slot);
  volatile int* tab = reinterpret_cast<volatile int*>(smem + SM::kItems);

  if (threadIdx.x == 0) {
    mbar_init(bar(SM::Q_FULL), 1); mbar_init(bar(SM::Q_FULL + 1), 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(bar(SM::K_FULL + s), 1); mbar_init(bar(SM::K_EMPTY + s), 1);
      mbar_init(bar(SM::V_FULL + s), 1); mbar_init(bar(SM::V_EMPTY + s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(SM::S_FULL + i), 1); mbar_init(bar(SM::P_FULL + i), 128); mbar_init(bar(SM::O_READY + i), 1);
      mbar_init(bar(SM::O_FREE + i), 128);
    }
    mbar_init(bar(SM::Q_EMPTY), 1);
    mbar_init(bar(SM::DONE), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_addr(tmem_slot), 512);
    tmem_relinquish();
  }
  if (warp == 2 || warp == 3) {
    // Block-list launches (one item per CTA): the first spare warp scans the lists of the query blocks under
    // each Q tile for the smallest and largest key block, 32 entries at a time.
    int bm_t0[2] = {0, 0}, bm_t1[2] = {0, 0};
    if (MASK == kRuntimeMods && p.bm_count && warp == 2) {
      int hb0;
      const int qt0 = fwd_slot_block(plan, blockIdx.x, 0, hb0);
#pragma unroll
      for (int X = 0; X < 2; ++X) {
        const int qx = qt0 * plan.rows + X * plan.q_step;
        int lo = 0x7fffffff, hi = -1;
        if (qx < p.Sq) {
          for (int qb = qx / p.bm_tm; qb <= (min(qx + BM, p.Sq) - 1) / p.bm_tm; ++qb) {
            const int nb = min(p.bm_count[qb], p.bm_stride);
            for (int t = lane; t < nb; t += 32) {
              const int j = p.bm_idx[(size_t)qb * p.bm_stride + t];
              lo = min(lo, j); hi = max(hi, j);
            }
          }
        }
        lo = __reduce_min_sync(0xffffffffu, lo); hi = __reduce_max_sync(0xffffffffu, hi);
        if (hi >= lo) { bm_t0[X] = lo * p.bm_tn / BN; bm_t1[X] = ((hi + 1) * p.bm_tn + BN - 1) / BN; }
      }
    }
    // the item table: thread k of the two spare warps works out item k
    const int k = threadIdx.x - 64;
    if (k < n_local) {
      volatile int* e = tab + k * IT_WORDS;
      int hb;
      const int slot = blockIdx.x + (k / plan.per_slot) * gridDim.x;
      const int qt = fwd_slot_block(plan, slot, k % plan.per_slot, hb);
      if (qt < 0) {
        e[IT_NTOT] = -1;                       // no such entry (middle block of an odd count)
      } else {
        const FwdItem it = fwd_item(p, plan, mask_flags, hb, qt, bm_t0, bm_t1);
#pragma unroll
        for (int X = 0; X < 2; ++X) {
          volatile int* w = e + X * WI_WORDS;
          w[WI_B] = it.b; w[WI_H] = it.h + X * plan.h_step; w[WI_Q0] = it.q0 + X * plan.q_step; w[WI_KLEN] = it.k_len;
          w[WI_QLIM] = it.q_lim; w[WI_KV0] = (it.jlo + it.tr[X].s) * BN; w[WI_N] = it.tr[X].e - it.tr[X].s;
          w[WI_RELEASE] = it.n_tot > 0;
        }
        e[IT_NTOT] = it.n_tot; e[IT_JLO] = it.jlo; e[IT_AS] = it.tr[0].s; e[IT_AE] = it.tr[0].e; e[IT_BS] = it.tr[1].s;
        e[IT_BE] = it.tr[1].e; e[IT_HK] = it.hk; e[IT_HEAD] = it.h; e[IT_Q0] = it.q0; e[IT_BATCH] = it.b;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Register split of the 384 x 168 pool: 4 x 32 x 96 + 8 x 32 x 200.  The producer and MMA-issuing
  // threads are on the latency-critical path of every hand-off and must not spill (measured on the
  // one-item form: 859 TFLOP/s with 56 registers against 944 with 88); the softmax rows fit in 200 once the
  // rare accumulator rescale is kept out of line.
  int k_loaded = 0, v_loaded = 0;   // producer thread only: K and V tiles it has asked for
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmO);
        bool ok = true;
        int ni = 0, g = 0;   // non-empty items and K/V tiles loaded so far (ring stage and phase)
        for (int k = 0; k < n_local && ok; ++k) {
          volatile int* e = tab + k * IT_WORDS;
          const int n_tot = e[IT_NTOT];
          if (n_tot <= 0) continue;
          const int jlo = e[IT_JLO], kvh = e[IT_BATCH] * p.Hkv + e[IT_HK];
          // One K/V tile of the item: waits for its ring stage, then asks for both halves.
          auto load_kv = [&](int j) {
            const int st = g % ST;
            const int row = (jlo + j) * BN;
            if (g >= ST) ok = mbar_wait(bar(SM::K_EMPTY + st), ((g / ST) - 1) & 1, abort_flag, &g_attn_fwd_status, 101);
            if (!ok) return;
            mbar_expect_tx(bar(SM::K_FULL + st), SM::kTile);
#pragma unroll
            for (int cc = 0; cc < DB / 128; ++cc)
              tma_load_3d(sbase + SM::kK + st * SM::kTile + cc * (BN * 128), &tmK, bar(SM::K_FULL + st), cc * kAtom, row, kvh);
            k_loaded = g + 1;
            if (g >= ST) ok = mbar_wait(bar(SM::V_EMPTY + st), ((g / ST) - 1) & 1, abort_flag, &g_attn_fwd_status, 102);
            if (!ok) return;
            mbar_expect_tx(bar(SM::V_FULL + st), SM::kTile);
#pragma unroll
            for (int cc = 0; cc < DB / 128; ++cc)
              tma_load_3d(sbase + SM::kV + st * SM::kTile + cc * (BN * 128), &tmV, bar(SM::V_FULL + st), cc * kAtom, row, kvh);
            v_loaded = g + 1;
            ++g;
          };
          // The item's first K/V tile goes out before its Q tiles: its ring stage frees a step before the
          // Q buffers do (those wait for the last Q K^T product of the item before), and the first
          // product of the new item needs both.
          load_kv(0);
          if (!ok) break;
          // both Q tiles (rows beyond Sq read as zeros), once every Q K^T product of the item before has run
          if (ni > 0) ok = mbar_wait(bar(SM::Q_EMPTY), (ni - 1) & 1, abort_flag, &g_attn_fwd_status, 103);
          if (!ok) break;
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            mbar_expect_tx(bar(SM::Q_FULL + X), SM::kTile);
#pragma unroll
            for (int cc = 0; cc < DB / 128; ++cc)
              tma_load_3d(sbase + SM::kQ + X * SM::kTile + cc * (BM * 128), &tmQ, bar(SM::Q_FULL + X), cc * kAtom,
                          e[IT_Q0] + X * plan.q_step, e[IT_BATCH] * p.H + e[IT_HEAD] + X * plan.h_step);
          }
          for (int j = 1; j < n_tot && ok; ++j) load_kv(j);
          ++ni;
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc_qk = idesc_f16(MmaFmt<T>::v, 0, 0, BM, BN);
        constexpr uint32_t idesc_pv = idesc_f16(MmaFmt<T>::v, 0, 1, BM, D);
        // Descriptors differ only in their 14-bit start-address field: build the constant upper
        // halves once and add a pre-shifted byte offset per MMA, so that the single issuing thread
        // spends a couple of integer instructions per tcgen05.mma instead of a dependent chain.
        const uint64_t dk_hi = smem_desc_sw128(0, 16, 1024);              // K-major Q / K operands
        // MN-major V operand: atoms of 8 rows x 128 bytes (16-bit) or 4 rows x 128 bytes in 32-byte units (TF32)
        const uint64_t dv_hi = kTf32 ? smem_desc_sw128_base32(0, BN * 128, 512) : smem_desc_sw128(0, BN * 128, 1024);
        auto desc_at = [](uint64_t hi, uint32_t saddr) { return hi | (uint64_t)((saddr & 0x3ffff) >> 4); };
        bool ok = true;
        int ni = 0, g0 = 0;      // non-empty items and K/V tiles of the items before this one
        int cb[2] = {0, 0};      // key tiles each Q tile took part in before this item (S / P / O phases)
        for (int k = 0; k < n_local && ok; ++k) {
          volatile int* e = tab + k * IT_WORDS;
          const int n_tot = e[IT_NTOT];
          if (n_tot <= 0) continue;
          const int ts[2] = {e[IT_AS], e[IT_BS]}, te[2] = {e[IT_AE], e[IT_BE]};
          auto active = [&](int X, int j) { return j >= ts[X] && j < te[X]; };
          auto issue_qk = [&](int X, int j) {
            const uint32_t d = tmem + X * 128;
            const uint64_t qd = desc_at(dk_hi, sbase + SM::kQ + X * SM::kTile);
            const uint64_t kd = desc_at(dk_hi, sbase + SM::kK + ((g0 + j) % ST) * SM::kTile);
#pragma unroll
            for (int kk = 0; kk < DB / 32; ++kk) {
              const uint32_t off = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4;   // compile-time constant
              mma_ss<kTf32>(d, qd + off, kd + off, idesc_qk, kk > 0);
            }
            tc_commit(bar(SM::S_FULL + X));
          };
          auto issue_pv = [&](int X, int j) {
            const uint32_t pa = tmem + X * 128;              // P: 64 columns of packed pairs (16-bit) or 128 of fp32 (TF32)
            const uint64_t vd = desc_at(dv_hi, sbase + SM::kV + ((g0 + j) % ST) * SM::kTile);
            const bool first = (j == ts[X]);
#pragma unroll
            for (int kk = 0; kk < BN / kKeysPerMma; ++kk)     // 8 columns of P and kKeysPerMma rows of V per step
              mma_ts<kTf32>(tmem + 256 + X * 128, pa + kk * 8, vd + (uint32_t)((kk * kKeysPerMma * 128) >> 4), idesc_pv,
                            !first || (kk > 0));
            tc_commit(bar(SM::O_READY + X));
          };
          ok = mbar_wait(bar(SM::Q_FULL + 0), ni & 1, abort_flag, &g_attn_fwd_status, 201);
          ok = ok && mbar_wait(bar(SM::Q_FULL + 1), ni & 1, abort_flag, &g_attn_fwd_status, 201);
          ok = ok && mbar_wait(bar(SM::K_FULL + g0 % ST), (g0 / ST) & 1, abort_flag, &g_attn_fwd_status, 202);
          if (!ok) break;
          tc_fence_after();
          if (active(0, 0)) issue_qk(0, 0);
          if (active(1, 0)) issue_qk(1, 0);
          tc_commit(bar(SM::K_EMPTY + g0 % ST));
          if (n_tot == 1) tc_commit(bar(SM::Q_EMPTY));
          for (int j = 0; j < n_tot && ok; ++j) {
            const int gj = g0 + j, st = gj % ST;
            bool v_ready = false, k_ready = false;
#pragma unroll
            for (int X = 0; X < 2; ++X) {
              if (active(X, j)) {
                if (!v_ready) { ok = mbar_wait(bar(SM::V_FULL + st), (gj / ST) & 1, abort_flag, &g_attn_fwd_status, 204); v_ready = true; }
                // the accumulator of the item before must have been read out before it is overwritten
                if (j == ts[X] && ni > 0)
                  ok = ok && mbar_wait(bar(SM::O_FREE + X), (ni - 1) & 1, abort_flag, &g_attn_fwd_status, 206);
                ok = ok && mbar_wait(bar(SM::P_FULL + X), (cb[X] + j - ts[X]) & 1, abort_flag, &g_attn_fwd_status, 205);
                if (!ok) break;
                tc_fence_after();
                issue_pv(X, j);
              }
              if (j + 1 < n_tot && active(X, j + 1)) {
                if (!k_ready) {
                  ok = mbar_wait(bar(SM::K_FULL + (gj + 1) % ST), ((gj + 1) / ST) & 1, abort_flag, &g_attn_fwd_status, 203);
                  k_ready = true;
                }
                if (!ok) break;
                tc_fence_after();
                issue_qk(X, j + 1);
              }
            }
            if (!ok) break;
            tc_commit(bar(SM::V_EMPTY + st));
            if (j + 1 < n_tot) {
              tc_commit(bar(SM::K_EMPTY + (gj + 1) % ST));
              if (j + 2 == n_tot) tc_commit(bar(SM::Q_EMPTY));   // every Q K^T product of the item is issued
            }
          }
          // a Q tile without keys in this item: keep in step with its warpgroup's O_FREE phases
#pragma unroll
          for (int X = 0; X < 2; ++X)
            if (ok && ni > 0 && te[X] == ts[X])
              ok = mbar_wait(bar(SM::O_FREE + X), (ni - 1) & 1, abort_flag, &g_attn_fwd_status, 207);
          cb[0] += te[0] - ts[0]; cb[1] += te[1] - ts[1];
          g0 += n_tot; ++ni;
        }
        // nothing may still be executing when the allocation is released
        tc_commit(bar(SM::DONE));
        mbar_drain(bar(SM::DONE), 0);
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int X = (warp >= 8) ? 1 : 0;
    bool ok = true;
    int ph = 0;      // key tiles this warpgroup walked in earlier items
    for (int k = 0; k < n_local && ok; ++k) {
      volatile const int* wi = tab + k * IT_WORDS + X * WI_WORDS;
      if (tab[k * IT_WORDS + IT_NTOT] < 0) continue;
      ok = softmax_tile<T, D, MASK, SCORE>(p, mask_flags, score_flags, X, wi, tmem, sbase, abort_flag, &tmO, Mout, Lout, ph, paired == 0);
      ph += wi[WI_N];
    }
    if (lane == 0) bulk_wait_read();      // the last boxes have left the staging buffer
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0 && lane == 0) {
    // make sure none of this CTA's TMA copies is still in flight before its shared memory is released
    for (int s = 0; s < ST; ++s) {
      // phase of the last tile that used stage s
      if (s < k_loaded) mbar_drain(bar(SM::K_FULL + s), (((k_loaded - 1 - s) / ST) ) & 1);
      if (s < v_loaded) mbar_drain(bar(SM::V_FULL + s), (((v_loaded - 1 - s) / ST) ) & 1);
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

// 3-D view (D, S, heads*batch) of a dense (D,S,H,B) array of 2- or 4-byte elements; box = one 128-byte swizzle
// atom x 128 rows x 1.  V with 4-byte elements is swizzled in 32-byte units (see smem_desc_sw128_base32).
// Output view for the epilogue's stores: box = 64 bytes x 32 rows, 64-byte swizzle.
static int32_t make_tmap_out(CUtensorMap* map, const void* base, int D, int S, int BH, int eb) {
  auto fn = encode_fn();
  TYLO_REQUIRE(fn, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)D * eb, (cuuint64_t)S * D * eb};
  cuuint32_t box[3] = {(cuuint32_t)(64 / eb), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, eb == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TYLO_REQUIRE(r == CUDA_SUCCESS, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult %d", (int)r);
  return TYLO_OK;
}

static int32_t make_tmap(CUtensorMap* map, const void* base, int D, int S, int BH, int eb, bool mn_major = false) {
  auto fn = encode_fn();
  TYLO_REQUIRE(fn, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)BH};
  cuuint64_t strides[2] = {(cuuint64_t)D * eb, (cuuint64_t)S * D * eb};
  cuuint32_t box[3] = {(cuuint32_t)(128 / eb), (cuuint32_t)BN, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, eb == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  (eb == 4 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TYLO_REQUIRE(r == CUDA_SUCCESS, TYLO_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return TYLO_OK;
}

bool attn_fwd_sm100_supported(const AttnParams& p, int32_t dtype) {
  if (dtype != TYLO_BF16 && dtype != TYLO_F16 && dtype != TYLO_F32_TF32) return false;
  // Head dims below the tile's run zero-padded (attention.jl:241-242): the TMA loads fill the columns beyond the
  // array with zeros and the stores clip them; a row must be a multiple of 16 bytes for the tensor maps.
  if (p.Dk != p.Dv || p.Dk < 8) return false;
  if (dtype == TYLO_F32_TF32 ? (p.Dk % 4 != 0 || p.Dk > 64) : (p.Dk % 8 != 0 || p.Dk > 128)) return false;
  if ((long long)p.Sq * p.H * p.B > 0x7fffffffLL / 2) return false;
  return true;
}

template <typename T, int D, uint32_t MASK, uint32_t SCORE>
static int32_t launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, float* M,
                          float* L, const AttnParams& p, cudaStream_t st) {
  auto kern = attn_fwd_sm100_kernel<T, D, MASK, SCORE>;
  TYLO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D * (int)sizeof(T)>::kDynamic));
  // One work item per CTA while the items fit the SMs in one go, and whenever the items' costs cannot be told
  // in advance (windows, document masks, ragged lengths: the hardware's own CTA scheduling balances those
  // best — measured on the window + document configuration: 0.337 ms against 0.346 ms).  Otherwise one CTA per
  // SM, each walking its share of the items with the next item's loads and first products under the previous
  // item's epilogue; under a causal-type mask a slot pairs a heavy with a light query block, so that every
  // CTA gets the same amount of work.
  const bool pair_heads = (p.G % 2) == 0;       // see FwdPlan: two heads of a group, or two row blocks of a head
  const long long nqt = pair_heads ? (p.Sq + BM - 1) / BM : (p.Sq + 2 * BM - 1) / (2 * BM);
  const long long heads = pair_heads ? p.H / 2 : p.H;
  const long long n_items = nqt * heads * p.B;
  const int sms = sm_count();
  const bool uneven = (p.mask_flags & (TYLO_MASK_SLIDING | TYLO_MASK_DOCUMENT | TYLO_MASK_PREFIX)) != 0 || p.k_lengths ||
                      p.q_lengths || p.n_or > 0 || p.bm_count;
  int paired = 0;
  long long grid = n_items;
  if (n_items > sms && !uneven) {
    paired = (p.mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_PREFIX_LM)) ? 2 : 1;
    const long long n_slots = (paired == 2 ? (nqt + 1) / 2 : nqt) * heads * p.B;
    grid = n_slots < sms ? n_slots : sms;
    const long long per_cta = kMaxItems / paired;                              // at most kMaxItems items per CTA
    const long long need = (n_slots + per_cta - 1) / per_cta;
    if (grid < need) grid = need;
  }
  kern<<<(unsigned)grid, kFwdThreads, FwdSmem<D * (int)sizeof(T)>::kDynamic, st>>>(mq, mk, mv, mo, M, L, p, paired);
  return check_launch("attn_fwd_sm100");
}

template <typename T, int D>
static int32_t dispatch_mods(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, float* M,
                             float* L, const AttnParams& p, cudaStream_t st) {
  constexpr uint32_t C = TYLO_MASK_CAUSAL, W = TYLO_MASK_SLIDING, DOC = TYLO_MASK_DOCUMENT;
  const uint32_t m = p.mask_flags, s = p.score_flags;
  if constexpr (sizeof(T) == 4) {
    // TF32: the plain and the causal forward have their own variants, every mod goes through the run-time one
    if (p.n_or == 0 && !p.bm_count && s == 0 && m == 0) return launch_fwd<T, D, 0, 0>(mq, mk, mv, mo, M, L, p, st);
    if (p.n_or == 0 && !p.bm_count && s == 0 && m == C) return launch_fwd<T, D, C, 0>(mq, mk, mv, mo, M, L, p, st);
    return launch_fwd<T, D, kRuntimeMods, kRuntimeMods>(mq, mk, mv, mo, M, L, p, st);
  } else {
  // OR-ed clauses, bias tables and block lists are handled by the variant that reads its flags at run time
  if (p.n_or > 0 || (s & TYLO_SCORE_BIAS) || p.bm_count) return launch_fwd<T, D, kRuntimeMods, kRuntimeMods>(mq, mk, mv, mo, M, L, p, st);
  if (s == 0) {
    if (m == 0) return launch_fwd<T, D, 0, 0>(mq, mk, mv, mo, M, L, p, st);
    if (m == C) return launch_fwd<T, D, C, 0>(mq, mk, mv, mo, M, L, p, st);
    if (m == (C | W) || m == W) return launch_fwd<T, D, W, 0>(mq, mk, mv, mo, M, L, p, st);
    if (m == (C | W | DOC) || m == (W | DOC)) return launch_fwd<T, D, W | DOC, 0>(mq, mk, mv, mo, M, L, p, st);
  }
  if (s == TYLO_SCORE_SOFTCAP && (m == (C | W | DOC) || m == (W | DOC)))
    return launch_fwd<T, D, W | DOC, TYLO_SCORE_SOFTCAP>(mq, mk, mv, mo, M, L, p, st);
  if (s == TYLO_SCORE_SOFTCAP && m == C) return launch_fwd<T, D, C, TYLO_SCORE_SOFTCAP>(mq, mk, mv, mo, M, L, p, st);
  if (s == TYLO_SCORE_ALIBI && m == C) return launch_fwd<T, D, C, TYLO_SCORE_ALIBI>(mq, mk, mv, mo, M, L, p, st);
  return launch_fwd<T, D, kRuntimeMods, kRuntimeMods>(mq, mk, mv, mo, M, L, p, st);
  }
}

int32_t attn_fwd_sm100(void* O, const void* Q, const void* K, const void* V, float* M, float* L, const AttnParams& p,
                       int32_t dtype, cudaStream_t st) {
  CUtensorMap mq, mk, mv, mo;
  const int eb = dtype == TYLO_F32_TF32 ? 4 : 2;
  if (int32_t rc = make_tmap_out(&mo, O, p.Dv, p.Sq, p.H * p.B, eb)) return rc;
  if (int32_t rc = make_tmap(&mq, Q, p.Dk, p.Sq, p.H * p.B, eb)) return rc;
  if (int32_t rc = make_tmap(&mk, K, p.Dk, p.Sk, p.Hkv * p.B, eb)) return rc;
  if (int32_t rc = make_tmap(&mv, V, p.Dv, p.Sk, p.Hkv * p.B, eb, true)) return rc;   // V is the MN-major operand of P V
  if (dtype == TYLO_F32_TF32) {
    if (p.Dk > 32) return dispatch_mods<float, 64>(mq, mk, mv, mo, M, L, p, st);
    return dispatch_mods<float, 32>(mq, mk, mv, mo, M, L, p, st);
  }
  if (dtype == TYLO_BF16) {
    if (p.Dk > 64) return dispatch_mods<__nv_bfloat16, 128>(mq, mk, mv, mo, M, L, p, st);
    return dispatch_mods<__nv_bfloat16, 64>(mq, mk, mv, mo, M, L, p, st);
  }
  if (p.Dk > 64) return dispatch_mods<__half, 128>(mq, mk, mv, mo, M, L, p, st);
  return dispatch_mods<__half, 64>(mq, mk, mv, mo, M, L, p, st);
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
