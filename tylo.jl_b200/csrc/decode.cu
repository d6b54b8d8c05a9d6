// Split-KV decode attention for sm_100a (decode_attention!, src/attention/decode.jl).
//
// The op is an HBM stream: every K and V row of the live cache is read exactly once and used
// by all G query heads of its KV head.  Per 512 bytes of K+V (head dim 128) that is 2*G*128
// multiply-adds, more than fp32 SIMT lanes can retire at HBM speed when G = 8, so the two
// small contractions run on tensor cores through warp-level mma (m16n8k16, fp32 accumulate)
// with the query group as the M dimension.  tcgen05 is not used here: its minimum M of 64
// would be 8x padding and the op is bandwidth bound either way.
//
// Layout of one CTA: NWARPS warps, each streaming its own K/V tiles of TN keys through a
// private cp.async ring (16-byte copies, XOR-swizzled rows, ldmatrix reads), each with its
// own online-softmax state, so the main loop has no CTA-wide barrier.  The warps' states are
// merged once at the end and the CTA writes one (normalised O, max, sum) partial.
//
// A scalar fp32 kernel covers fp32 storage and any shape the tensor path does not.
#include <type_traits>

#include "common.cuh"
#include "decode_merge.cuh"

namespace tylo {

constexpr float kLog2eD = 1.4426950408889634f;

// ---- small PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: nothing is read, 16 zero bytes are written
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 p = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

// ---- one-launch tail ---------------------------------------------------------------------------------
// With a ticket buffer the split kernel also finishes the job: CTAs draw a ticket per group of kGroup
// consecutive splits of their (kv head, batch); the CTA that completes a group folds the group's partials
// into one (written over the group's first slot), then draws a second-level ticket; the CTA that
// completes the last group merges the group partials and writes O — or, when the sequence is sharded
// over GPUs, pushes the merged record to every peer, waits (bounded) for theirs and merges those.
// The merge algebra is mha_decode_combine's (decode.jl:119-140).  Every counter is put back to zero by
// the CTA that completes it, so a zeroed buffer stays valid from call to call.
constexpr int kGroup = 8;

struct DecodeTail {
  int32_t* tickets;              // null: write the partials only
  void* O;                       // (Dv, H, B) in the storage type
  ExchangePeers peers;           // receive buffers of all ranks (world > 1)
  int rank, world;
  unsigned long long timeout_ns;
};

// Paged KV cache: K and V are pools of pages of `page_size` keys, laid out (D, page_size, Hkv, n_pages);
// sequence b's keys [i * page_size, (i + 1) * page_size) live in page table[b * max_pages + i].
struct DecodePages {
  const int32_t* table;          // null: K, V are dense (D, Sk, Hkv, B) arrays
  int page_size, max_pages;
};

__host__ __device__ inline int decode_groups(int n_splits) { return (n_splits + kGroup - 1) / kGroup; }

// One warp merges `count` partials of head `hb` (slots first, first + step, ...): lane owns VEC = D / 32
// adjacent columns.  All loads of a round are independent; they go to L2 (written by other CTAs).
template <int D>
__device__ __forceinline__ void merge_slots(const float* Op, const float* Mp, const float* Lp, size_t BH, size_t hb,
                                            int first, int step, int count, int lane, float (&o)[D / 32], float& m_out,
                                            float& l_out) {
  constexpr int VEC = D / 32;
  float m = -INFINITY;
  for (int k = lane; k < count; k += 32) m = fmaxf(m, __ldcg(Mp + (size_t)(first + k * step) * BH + hb));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  float l = 0.f;
  for (int k0 = 0; k0 < count; k0 += kGroup) {
    float ms[kGroup], ls[kGroup], val[kGroup][VEC];
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      const bool live = k0 + u < count;
      const size_t slot = ((size_t)(first + (live ? k0 + u : 0) * step)) * BH + hb;
      ms[u] = live ? __ldcg(Mp + slot) : -INFINITY;
      ls[u] = live ? __ldcg(Lp + slot) : 0.f;
      if (VEC == 4) {
        const float4 t = live ? __ldcg(reinterpret_cast<const float4*>(Op + slot * D) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        val[u][0] = t.x; val[u][1] = t.y; val[u][VEC - 2] = t.z; val[u][VEC - 1] = t.w;
      } else {
        const float2 t = live ? __ldcg(reinterpret_cast<const float2*>(Op + slot * D) + lane) : make_float2(0.f, 0.f);
        val[u][0] = t.x; val[u][1] = t.y;
      }
    }
#pragma unroll
    for (int u = 0; u < kGroup; ++u) {
      const float w = (ms[u] == -INFINITY) ? 0.f : ls[u] * exp2f(ms[u] - m);
      l += w;
#pragma unroll
      for (int v = 0; v < VEC; ++v) acc[v] += w * val[u][v];
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int v = 0; v < VEC; ++v) o[v] = acc[v] * inv;
  m_out = m; l_out = l;
}

// The same merge over the records the ranks of a sharded sequence have pushed into this GPU's receive
// buffer: record r starts `stride` words after record r - 1 and holds D values, the max and the sum.
template <int D>
__device__ __forceinline__ void merge_records(const float* recs, int64_t stride, int count, int lane, float (&o)[D / 32],
                                              float& m_out, float& l_out) {
  constexpr int VEC = D / 32;
  float m = -INFINITY;
  for (int r = 0; r < count; ++r) m = fmaxf(m, __ldcg(recs + r * stride + D));
  float acc[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
  float l = 0.f;
#pragma unroll 4
  for (int r = 0; r < count; ++r) {
    const float* rec = recs + r * stride;
    const float mr = __ldcg(rec + D), lr = __ldcg(rec + D + 1);
    const float w = (mr == -INFINITY) ? 0.f : lr * exp2f(mr - m);
    l += w;
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] += w * __ldcg(rec + lane * VEC + v);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int v = 0; v < VEC; ++v) o[v] = acc[v] * inv;
  m_out = m; l_out = l;
}

template <int D>
__device__ __forceinline__ void store_row(float* dst, int lane, const float (&o)[D / 32]) {
  if (D / 32 == 4) reinterpret_cast<float4*>(dst)[lane] = make_float4(o[0], o[1], o[D / 32 - 2], o[D / 32 - 1]);
  else reinterpret_cast<float2*>(dst)[lane] = make_float2(o[0], o[1]);
}

// Tail of one (kv head, batch) CTA after its own partial is in memory.  Uniform over the CTA.
template <typename T, int D, int NWARPS>
__device__ __forceinline__ void decode_tail(const DecodeTail& tail, float* Op, float* Mp, float* Lp, int n_splits,
                                            int split, int hkb, int b, int hk, int H, int B, int G) {
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_groups = decode_groups(n_splits);
  const int gi = split / kGroup;
  const int gfirst = gi * kGroup;
  const int gsz = min(kGroup, n_splits - gfirst);
  int32_t* tk = tail.tickets + (size_t)hkb * (n_groups + 1);
  const size_t BH = (size_t)B * H;

  // ---- level 1: the CTA that completes its group folds the group into slot `gfirst` --------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&tk[gi], 1);
    s_last = (t == gsz - 1);
    if (s_last) tk[gi] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (gsz > 1) {
    for (int g = warp; g < G; g += NWARPS) {
      const size_t hb = (size_t)b * H + (size_t)hk * G + g;
      float o[D / 32], m, l;
      merge_slots<D>(Op, Mp, Lp, BH, hb, gfirst, 1, gsz, lane, o, m, l);
      __syncwarp();
      const size_t slot = (size_t)gfirst * BH + hb;
      store_row<D>(Op + slot * D, lane, o);
      if (lane == 0) { Mp[slot] = m; Lp[slot] = l; }
    }
  }

  // ---- level 2: the CTA that completes the last group merges the group partials -----------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(&tk[n_groups], 1);
    s_last = (t == n_groups - 1);
    if (s_last) tk[n_groups] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  T* O = static_cast<T*>(tail.O);
  const int world = tail.world, rank = tail.rank;
  const ExchangeLayout lay = exchange_layout(world, (int)BH, D);
  constexpr int kHeadsPerWarp = 16 / NWARPS;      // G <= 16
  float o[kHeadsPerWarp][D / 32], m[kHeadsPerWarp], l[kHeadsPerWarp];
  uint32_t epoch[kHeadsPerWarp];
  uint32_t* self = reinterpret_cast<uint32_t*>(tail.peers.buf[rank]);

  // this GPU's record of each of the warp's heads; with peers, pushed to every rank (its own buffer included)
#pragma unroll
  for (int k = 0; k < kHeadsPerWarp; ++k) {
    const int g = warp + k * NWARPS;
    if (g >= G) break;
    const size_t hb = (size_t)b * H + (size_t)hk * G + g;
    merge_slots<D>(Op, Mp, Lp, BH, hb, 0, kGroup, n_groups, lane, o[k], m[k], l[k]);
    if (world > 1) {
      epoch[k] = self[lay.epoch_off + hb] + 1u;     // call counter of this head
      const int par = (int)(epoch[k] & 1u);
      for (int p = 0; p < world; ++p) {
        float* rec = tail.peers.buf[p] + lay.data_off + ((int64_t)(par * world + rank) * (int64_t)BH + (int64_t)hb) * lay.rec;
        store_row<D>(rec, lane, o[k]);
        if (lane == 0) *reinterpret_cast<float2*>(rec + D) = make_float2(m[k], l[k]);
      }
    }
  }
  if (world > 1) {
    // One fence for all of the warp's records: every lane's peer stores are ordered before the flags raised
    // below, then one round of flags and one round of (bounded) waits.
    __threadfence_system();
    __syncwarp();
#pragma unroll
    for (int k = 0; k < kHeadsPerWarp; ++k) {
      const int g = warp + k * NWARPS;
      if (g >= G) break;
      const size_t hb = (size_t)b * H + (size_t)hk * G + g;
      if (lane < world)
        st_release_sys(reinterpret_cast<uint32_t*>(tail.peers.buf[lane]) + lay.flag_off + (int64_t)rank * (int64_t)BH + (int64_t)hb, epoch[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < kHeadsPerWarp; ++k) {
    const int g = warp + k * NWARPS;
    if (g >= G) break;
    const size_t hb = (size_t)b * H + (size_t)hk * G + g;
    if (world > 1) {
      bool ok = true;
      if (lane < world) {
        const uint32_t* f = self + lay.flag_off + (int64_t)lane * (int64_t)BH + (int64_t)hb;
        const unsigned long long t0 = global_ns();
        while ((int32_t)(ld_acquire_sys(f) - epoch[k]) < 0) {          // bounded wait for rank `lane`'s record
          if (global_ns() - t0 > tail.timeout_ns) { ok = false; break; }
          __nanosleep(64);
        }
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        // a peer never arrived: record it, keep the call counter in step, leave O untouched
        if (lane == 0) { atomicMax(self, 1u + (uint32_t)hb); self[lay.epoch_off + hb] = epoch[k]; }
        continue;
      }
      const int par = (int)(epoch[k] & 1u);
      const float* recs = tail.peers.buf[rank] + lay.data_off + ((int64_t)par * world * (int64_t)BH + (int64_t)hb) * lay.rec;
      merge_records<D>(recs, (int64_t)BH * lay.rec, world, lane, o[k], m[k], l[k]);
      if (lane == 0) self[lay.epoch_off + hb] = epoch[k];
    }
    // output in the storage type
    T* dst = O + hb * D + lane * (D / 32);
#pragma unroll
    for (int v = 0; v < D / 32; ++v) dst[v] = Elem<T>::from_f(o[k][v]);
  }
}

// ---- tensor path ----------------------------------------------------------------------------------
// grid.x = n_splits * Hkv * B, split fastest.  G16: query group of 9..16 heads (rows 8..15 live).
template <typename T, int D, int TN, int NWARPS, int STAGES, bool G16, bool PAGED>
__global__ void __launch_bounds__(NWARPS * 32)
decode_split_mma_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                        const int32_t* __restrict__ lengths, float* __restrict__ Op,
                        float* __restrict__ Mp, float* __restrict__ Lp, int Sk, int H, int Hkv, int B,
                        int G, int n_splits, int split_size, float scale_log2,
                        const __grid_constant__ DecodeTail tail, const __grid_constant__ DecodePages pages) {
  constexpr int ROW_BYTES = D * 2;
  constexpr int CHUNKS = ROW_BYTES / 16;          // 16-byte chunks per row
  constexpr int TILE_BYTES = TN * ROW_BYTES;      // one K (or V) tile
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = TN / 8;                      // n8 tiles of S per tile
  constexpr int DT = D / 8;                       // n8 tiles of O
  static_assert(WARP_BYTES >= 16 * D * 4 + 128, "merge staging must fit in the warp's ring");
  extern __shared__ __align__(128) uint8_t smem[];

  // This kernel may have been placed while the launch before it on the stream was still finishing
  // (programmatic dependent launch).  It streams its keys and values straight away and waits for that
  // launch only before its first write to memory the two may share (partials, tickets, output): Q, K, V
  // must therefore not be produced by a decode launch of this library directly ahead on the stream.
  dependents_may_launch();   // whatever follows may be placed while the splits still run
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x % n_splits;
  const int hkb = blockIdx.x / n_splits;
  const int b = hkb / Hkv, hk = hkb % Hkv;
  int len = lengths[b];
  len = len < 0 ? 0 : (len > Sk ? Sk : len);
  const int begin = split * split_size;
  int end = begin + split_size; if (end > len) end = len;
  const int ntiles = end > begin ? (end - begin + TN - 1) / TN : 0;
  const int my_tiles = ntiles > warp ? (ntiles - warp + NWARPS - 1) / NWARPS : 0;

  uint8_t* wsm = smem + warp * WARP_BYTES;
  const uint32_t wsm_u = smem_u32(wsm);
  const T* kbase_g = K + ((size_t)(b * Hkv + hk) * Sk) * D;
  const T* vbase_g = V + ((size_t)(b * Hkv + hk) * Sk) * D;
  const int32_t* page_row = PAGED ? pages.table + (size_t)b * pages.max_pages : nullptr;

  auto issue = [&](int i) {
    const int tile = warp + i * NWARPS;
    const int kv0 = begin + tile * TN;
    const uint32_t st = wsm_u + (i % STAGES) * STAGE_BYTES;
    // a tile never straddles pages (page_size is a multiple of the tile): one table look-up per tile
    const T* kt = kbase_g; const T* vt = vbase_g;
    int kv_off = 0;
    if (PAGED) {
      const int pg = __ldg(page_row + kv0 / pages.page_size);
      const size_t pbase = ((size_t)pg * Hkv + hk) * pages.page_size * D;
      kt = K + pbase; vt = V + pbase;
      kv_off = (kv0 / pages.page_size) * pages.page_size;
    }
#pragma unroll
    for (int c = 0; c < TN * CHUNKS / 32; ++c) {
      const int idx = c * 32 + lane;
      const int row = idx / CHUNKS, chunk = idx % CHUNKS;
      const int kv = kv0 + row;
      const bool ok = kv < end;
      const size_t goff = (size_t)((ok ? kv : kv0) - kv_off) * D + chunk * 8;
      const uint32_t soff = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
      cp_async16(st + soff, kt + goff, ok);
      cp_async16(st + TILE_BYTES + soff, vt + goff, ok);
    }
  };

  // Q fragments (A operand, rows = heads of the group, zero padded)
  uint32_t qa[KSTEPS][4];
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    const T* q0 = Q + ((size_t)b * H + (size_t)hk * G + r0) * D;
    const T* q1 = q0 + (size_t)8 * D;
    const bool v0 = r0 < G, v1 = G16 && (r0 + 8 < G);
#pragma unroll
    for (int t = 0; t < KSTEPS; ++t) {
      qa[t][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + t * 16 + c0) : 0u;
      qa[t][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + t * 16 + c0 + 8) : 0u;
      qa[t][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + t * 16 + c0) : 0u;
      qa[t][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + t * 16 + c0 + 8) : 0u;
    }
  }

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < my_tiles) issue(i);
    cp_async_commit();
  }

  for (int i = 0; i < my_tiles; ++i) {
    cp_async_wait<STAGES - 2>();
    __syncwarp();
    if (i + STAGES - 1 < my_tiles) issue(i + STAGES - 1);
    cp_async_commit();

    const uint32_t kst = wsm_u + (i % STAGES) * STAGE_BYTES;
    const uint32_t vst = kst + TILE_BYTES;
    const int kv0 = begin + (warp + i * NWARPS) * TN;

    // S = Q K^T
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
    for (int t2 = 0; t2 < KSTEPS / 2; ++t2) {
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int row = j * 8 + (lane & 7);
        const int chunk = 4 * t2 + (lane >> 3);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kst + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), b0, b1, b2, b3);
        mma16816<T>(s[j], qa[2 * t2], b0, b1);
        mma16816<T>(s[j], qa[2 * t2 + 1], b2, b3);
      }
    }
    // scale, mask the ragged tail
    const bool tail = kv0 + TN > end;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int col = kv0 + j * 8 + (lane & 3) * 2;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[j][e] * scale_log2;
        if (tail && col + (e & 1) >= end) v = -INFINITY;
        s[j][e] = v;
      }
    }
    // online softmax (row r0 = lane/4 in regs 0,1; row r0+8 in regs 2,3)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      if (G16) mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    if (G16) {
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    }
    const float mn0 = fmaxf(m0, mx0);           // finite: every tile holds at least one live key
    const float mn1 = G16 ? fmaxf(m1, mx1) : 0.f;
    const float a0 = exp2f(m0 - mn0);
    const float a1 = G16 ? exp2f(m1 - mn1) : 0.f;
    m0 = mn0; m1 = G16 ? mn1 : m1;
    float ps0 = 0.f, ps1 = 0.f;
    uint32_t pa[NT / 2][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const float p0 = exp2f(s[j][0] - mn0), p1 = exp2f(s[j][1] - mn0);
      const float p2 = G16 ? exp2f(s[j][2] - mn1) : 0.f, p3 = G16 ? exp2f(s[j][3] - mn1) : 0.f;
      ps0 += p0 + p1; ps1 += p2 + p3;
      pa[j / 2][(j & 1) * 2 + 0] = pack2<T>(p0, p1);
      pa[j / 2][(j & 1) * 2 + 1] = pack2<T>(p2, p3);
    }
    l0 = l0 * a0 + ps0;
    l1 = l1 * a1 + ps1;
#pragma unroll
    for (int i2 = 0; i2 < DT; ++i2) {
      o[i2][0] *= a0; o[i2][1] *= a0;
      if (G16) { o[i2][2] *= a1; o[i2][3] *= a1; }
    }
    // O += P V
#pragma unroll
    for (int u = 0; u < TN / 16; ++u) {
#pragma unroll
      for (int ii = 0; ii < DT / 2; ++ii) {
        const int q = lane >> 3;
        const int row = 16 * u + (q & 1) * 8 + (lane & 7);
        const int chunk = 2 * ii + (q >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(vst + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4), b0, b1, b2, b3);
        mma16816<T>(o[2 * ii], pa[u], b0, b1);
        mma16816<T>(o[2 * ii + 1], pa[u], b2, b3);
      }
    }
  }
  cp_async_wait<0>();
  __syncwarp();

  // finish the row sums over the quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

  // stage this warp's state in its own ring: O[16][D] fp32, then m[16], l[16]
  float* so = reinterpret_cast<float*>(wsm);
  float* sm = so + 16 * D;
  float* sl = sm + 16;
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int i2 = 0; i2 < DT; ++i2) {
      *reinterpret_cast<float2*>(so + r0 * D + i2 * 8 + c0) = make_float2(o[i2][0], o[i2][1]);
      if (G16) *reinterpret_cast<float2*>(so + (r0 + 8) * D + i2 * 8 + c0) = make_float2(o[i2][2], o[i2][3]);
    }
    if ((lane & 3) == 0) {
      sm[r0] = m0; sl[r0] = l0;
      sm[r0 + 8] = G16 ? m1 : -INFINITY; sl[r0 + 8] = G16 ? l1 : 0.f;
    }
  }
  __syncthreads();
  dependency_wait();

  // merge the warps and write the split's partial
  for (int idx = threadIdx.x; idx < G * D; idx += NWARPS * 32) {
    const int g = idx / D, d = idx % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) m = fmaxf(m, reinterpret_cast<const float*>(smem + w * WARP_BYTES)[16 * D + g]);
    float acc = 0.f, l = 0.f;
    if (m != -INFINITY) {
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        const float* wo = reinterpret_cast<const float*>(smem + w * WARP_BYTES);
        const float f = exp2f(wo[16 * D + g] - m);
        acc += wo[g * D + d] * f;
        l += wo[16 * D + 16 + g] * f;
      }
    }
    const size_t hb = (size_t)split * B * H + (size_t)b * H + (size_t)hk * G + g;
    Op[hb * D + d] = l > 0.f ? acc / l : 0.f;
    if (d == 0) { Mp[hb] = m; Lp[hb] = l; }
  }
  if (tail.tickets) decode_tail<T, D, NWARPS>(tail, Op, Mp, Lp, n_splits, split, hkb, b, hk, H, B, G);
}

// ---- scalar path: any dtype, D <= 512, any G ----------------------------------------------------
// grid.x = n_splits * H * B (split fastest); 4 warps, each striding over the split's keys.
template <typename T>
__global__ void __launch_bounds__(128)
decode_split_generic_kernel(const T* __restrict__ Q, const T* __restrict__ K, const T* __restrict__ V,
                            const int32_t* __restrict__ lengths, float* __restrict__ Op,
                            float* __restrict__ Mp, float* __restrict__ Lp, int Dk, int Dv, int Sk,
                            int H, int Hkv, int B, int G, int n_splits, int split_size, float scale_log2) {
  constexpr int MAXR = 16;  // per-lane slice of the head dim (D <= 512)
  __shared__ float sacc[4][512];
  __shared__ float sm[4], sl[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x % n_splits;
  const int hb = blockIdx.x / n_splits;
  const int b = hb / H, h = hb % H, hk = h / G;
  int len = lengths[b];
  len = len < 0 ? 0 : (len > Sk ? Sk : len);
  const int begin = split * split_size;
  int end = begin + split_size; if (end > len) end = len;

  float q[MAXR], acc[MAXR];
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int d = r * 32 + lane;
    q[r] = d < Dk ? Elem<T>::to_f(Q[((size_t)b * H + h) * Dk + d]) : 0.f;
    acc[r] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const T* kb = K + ((size_t)(b * Hkv + hk) * Sk) * Dk;
  const T* vb = V + ((size_t)(b * Hkv + hk) * Sk) * Dv;
  for (int kv = begin + warp; kv < end; kv += 4) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      const int d = r * 32 + lane;
      if (d < Dk) s += q[r] * Elem<T>::to_f(kb[(size_t)kv * Dk + d]);
    }
    s = warp_reduce(s, SumOp()) * scale_log2;
    const float mn = fmaxf(m, s);
    const float a = exp2f(m - mn), p = exp2f(s - mn);
    l = l * a + p; m = mn;
#pragma unroll
    for (int r = 0; r < MAXR; ++r) {
      const int d = r * 32 + lane;
      if (d < Dv) acc[r] = acc[r] * a + p * Elem<T>::to_f(vb[(size_t)kv * Dv + d]);
    }
  }
#pragma unroll
  for (int r = 0; r < MAXR; ++r) {
    const int d = r * 32 + lane;
    if (d < Dv) sacc[warp][d] = acc[r];
  }
  if (lane == 0) { sm[warp] = m; sl[warp] = l; }
  __syncthreads();
  float mg = fmaxf(fmaxf(sm[0], sm[1]), fmaxf(sm[2], sm[3]));
  float f[4], lg = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) { f[w] = mg == -INFINITY ? 0.f : exp2f(sm[w] - mg); lg += sl[w] * f[w]; }
  const size_t out = (size_t)split * B * H + (size_t)b * H + h;
  for (int d = threadIdx.x; d < Dv; d += 128) {
    const float a = sacc[0][d] * f[0] + sacc[1][d] * f[1] + sacc[2][d] * f[2] + sacc[3][d] * f[3];
    Op[out * Dv + d] = lg > 0.f ? a / lg : 0.f;
  }
  if (threadIdx.x == 0) { Mp[out] = mg; Lp[out] = lg; }
}

// ---- combine --------------------------------------------------------------------------------------
// One CTA per (head, batch): SL split-lanes x Dv columns.  Two-pass form of the reference's
// sequential merge (decode.jl:119-140): weights l_s * exp2(m_s - max_s m_s), guarded for -Inf.
template <typename T, int SL>
__global__ void __launch_bounds__(1024)
decode_combine_kernel(T* __restrict__ O, float* __restrict__ Om, float* __restrict__ Mm, float* __restrict__ Lm,
                      const float* __restrict__ Op, const float* __restrict__ Mp, const float* __restrict__ Lp,
                      int n_splits, int64_t o_stride, int64_t ml_stride, int Dv) {
  extern __shared__ float csm[];  // [SL][Dv] accumulators, then [SL] sums
  const int hb = blockIdx.x;
  const int sl = threadIdx.y;
  float m = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, Mp[(size_t)s * ml_stride + hb]);
  float lsum = 0.f;
  for (int d0 = 0; d0 < Dv; d0 += blockDim.x) {
    const int d = d0 + threadIdx.x;
    float acc = 0.f; lsum = 0.f;
    for (int s = sl; s < n_splits; s += SL) {
      const float ms = Mp[(size_t)s * ml_stride + hb];
      const float w = (m == -INFINITY) ? 0.f : Lp[(size_t)s * ml_stride + hb] * exp2f(ms - m);
      lsum += w;
      if (d < Dv && w != 0.f) acc += w * Op[(size_t)s * o_stride + (size_t)hb * Dv + d];
    }
    if (d < Dv) csm[sl * Dv + d] = acc;
  }
  if (threadIdx.x == 0) csm[SL * Dv + sl] = lsum;
  __syncthreads();
  if (sl == 0) {
    float l = 0.f;
#pragma unroll
    for (int k = 0; k < SL; ++k) l += csm[SL * Dv + k];
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < SL; ++k) acc += csm[k * Dv + d];
      const float r = l > 0.f ? acc / l : 0.f;
      if (O) O[(size_t)hb * Dv + d] = Elem<T>::from_f(r);
      if (Om) Om[(size_t)hb * Dv + d] = r;
    }
    if (threadIdx.x == 0 && Mm) { Mm[hb] = m; Lm[hb] = l; }
  }
}

// Block-parallel form (Dv % 4 == 0, 16-byte aligned partials): 1024 threads fold the partials with
// independent vector loads, see merge_partials.
template <typename T>
__global__ void __launch_bounds__(1024)
decode_combine_wide_kernel(T* __restrict__ O, float* __restrict__ Om, float* __restrict__ Mm, float* __restrict__ Lm,
                           const float* __restrict__ Op, const float* __restrict__ Mp, const float* __restrict__ Lp,
                           int n_splits, int64_t o_stride, int64_t ml_stride, int Dv) {
  extern __shared__ __align__(16) float wsm[];
  float* res = wsm + 4096 + 64;
  const int hb = blockIdx.x;
  const int tid = threadIdx.y * blockDim.x + threadIdx.x;
  dependency_wait();
  dependents_may_launch();
  float m, l;
  merge_partials<false>(Op + (size_t)hb * Dv, Mp + hb, Lp + hb, n_splits, o_stride, ml_stride, Dv, wsm, res, m, l);
  if (tid < Dv) {
    if (O) O[(size_t)hb * Dv + tid] = Elem<T>::from_f(res[tid]);
    if (Om) Om[(size_t)hb * Dv + tid] = res[tid];
  }
  if (tid == 0 && Mm) { Mm[hb] = m; Lm[hb] = l; }
}

// ---- host side --------------------------------------------------------------------------------------
static int decode_split_size(int Sk, int n_splits) {
  const int per = (Sk + n_splits - 1) / n_splits;
  return ((per + 63) / 64) * 64;  // decode.jl:183 with TILE_N = 64
}

template <typename T, int D, int TN, int NWARPS, int STAGES>
static int32_t launch_decode_mma(const void* Q, const void* K, const void* V, const int32_t* lengths, float* Op,
                                 float* Mp, float* Lp, int n_splits, int Sk, int H, int Hkv, int B,
                                 const DecodeTail& tail, const DecodePages& pages, cudaStream_t st) {
  const int G = H / Hkv;
  const int split_size = decode_split_size(Sk, n_splits);
  const float scale_log2 = kLog2eD / sqrtf((float)D);
  constexpr int SMEM = NWARPS * STAGES * 2 * TN * D * 2;
  const unsigned grid = (unsigned)((int64_t)n_splits * Hkv * B);
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return e;
    return launch_overlapped(true, kern, dim3(grid), dim3(NWARPS * 32), SMEM, st, (const T*)Q, (const T*)K, (const T*)V, lengths,
                             Op, Mp, Lp, Sk, H, Hkv, B, G, n_splits, split_size, scale_log2, tail, pages);
  };
  const bool paged = pages.table != nullptr;
  if (G <= 8) {
    if (paged) TYLO_CUDA_OK(go(decode_split_mma_kernel<T, D, TN, NWARPS, STAGES, false, true>));
    else TYLO_CUDA_OK(go(decode_split_mma_kernel<T, D, TN, NWARPS, STAGES, false, false>));
  } else {
    if (paged) TYLO_CUDA_OK(go(decode_split_mma_kernel<T, D, TN, NWARPS, STAGES, true, true>));
    else TYLO_CUDA_OK(go(decode_split_mma_kernel<T, D, TN, NWARPS, STAGES, true, false>));
  }
  return check_launch("decode_split_mma");
}

// Whether the tensor-core split kernel (and with it the one-launch tail) covers these extents.
static bool decode_mma_eligible(int32_t dtype, int Dk, int Dv, int H, int Hkv) {
  return (dtype == TYLO_BF16 || dtype == TYLO_F16) && Dk == Dv && (Dk == 64 || Dk == 128) && Hkv > 0 && H / Hkv <= 16;
}

template <typename T>
static int32_t decode_split_dispatch(const void* Q, const void* K, const void* V, const int32_t* lengths,
                                     float* Op, float* Mp, float* Lp, int n_splits, int Dk, int Dv, int Sk,
                                     int H, int Hkv, int B, const DecodeTail& tail, const DecodePages& pages,
                                     cudaStream_t st) {
  const int G = H / Hkv;
  if constexpr (!std::is_same<T, float>::value) {
    if (Dk == Dv && (Dk == 64 || Dk == 128) && G <= 16) {
      // 16-key tiles at head dim 128 (96 KB of rings, two CTAs per SM), 32-key tiles at 64: the best of the
      // tile / stage combinations measured (32-key tiles with 3 stages leave one CTA per SM at D 128).
      if (Dk == 128) return launch_decode_mma<T, 128, 16, 4, 3>(Q, K, V, lengths, Op, Mp, Lp, n_splits, Sk, H, Hkv, B, tail, pages, st);
      return launch_decode_mma<T, 64, 32, 4, 3>(Q, K, V, lengths, Op, Mp, Lp, n_splits, Sk, H, Hkv, B, tail, pages, st);
    }
  }
  TYLO_REQUIRE(tail.tickets == nullptr, TYLO_ERR_UNSUPPORTED, "decode: the one-launch form needs the tensor-core split kernel");
  TYLO_REQUIRE(pages.table == nullptr, TYLO_ERR_UNSUPPORTED,
               "decode: a paged cache needs 16-bit storage, head dim 64 or 128 and at most 16 query heads per kv head");
  TYLO_REQUIRE(Dk <= 512 && Dv <= 512, TYLO_ERR_UNSUPPORTED, "decode: head dims above 512 are not supported");
  const int split_size = decode_split_size(Sk, n_splits);
  const float scale_log2 = kLog2eD / sqrtf((float)Dk);
  const unsigned grid = (unsigned)((int64_t)n_splits * H * B);
  decode_split_generic_kernel<T><<<grid, 128, 0, st>>>((const T*)Q, (const T*)K, (const T*)V, lengths, Op, Mp, Lp,
                                                       Dk, Dv, Sk, H, Hkv, B, G, n_splits, split_size, scale_log2);
  return check_launch("decode_split_generic");
}

template <typename T>
static int32_t decode_combine_dispatch(void* O, float* Om, float* Mm, float* Lm, const float* Op, const float* Mp,
                                       const float* Lp, int n_splits, int64_t o_stride, int64_t ml_stride, int Dv,
                                       int H, int B, cudaStream_t st) {
  const int tx = Dv >= 128 ? 128 : (Dv >= 64 ? 64 : 32);
  const unsigned grid = (unsigned)((int64_t)H * B);
  // Many partials per head (long contexts): the 1024-thread block-parallel merge.  Few partials: a small
  // block per head, or a thousand mostly idle threads per head would cost more than the merge itself.
  if (n_splits > 16 && Dv % 4 == 0 && Dv <= 512 && aligned16(Op) && o_stride % 4 == 0) {
    TYLO_CUDA_OK(launch_overlapped(true, decode_combine_wide_kernel<T>, dim3(grid), merge_block(Dv),
                                   merge_smem_floats(1024, Dv) * sizeof(float), st, (T*)O, Om, Mm, Lm, Op, Mp, Lp,
                                   n_splits, o_stride, ml_stride, Dv));
    return check_launch("decode_combine_wide");
  }
  if (n_splits > 8) {
    constexpr int SL = 8;
    decode_combine_kernel<T, SL><<<grid, dim3(tx, SL), (SL * Dv + SL) * sizeof(float), st>>>(
        (T*)O, Om, Mm, Lm, Op, Mp, Lp, n_splits, o_stride, ml_stride, Dv);
  } else {
    constexpr int SL = 2;
    decode_combine_kernel<T, SL><<<grid, dim3(tx, SL), (SL * Dv + SL) * sizeof(float), st>>>(
        (T*)O, Om, Mm, Lm, Op, Mp, Lp, n_splits, o_stride, ml_stride, Dv);
  }
  return check_launch("decode_combine");
}

static int32_t check_decode_dims(const char* who, int n_splits, int Dk, int Dv, int Sk, int H, int Hkv, int B) {
  TYLO_REQUIRE(Dk > 0 && Dv > 0 && Sk > 0 && H > 0 && Hkv > 0 && B > 0, TYLO_ERR_INVALID_ARGUMENT,
               "%s: extents must be positive (Dk=%d Dv=%d Sk=%d H=%d Hkv=%d B=%d)", who, Dk, Dv, Sk, H, Hkv, B);
  TYLO_REQUIRE(H % Hkv == 0, TYLO_ERR_INVALID_ARGUMENT, "%s: Heads (%d) must be a multiple of Heads_KV (%d)", who,
               H, Hkv);
  TYLO_REQUIRE(n_splits > 0, TYLO_ERR_INVALID_ARGUMENT, "%s: n_splits must be positive", who);
  TYLO_REQUIRE((int64_t)n_splits * H * B <= 0x7fffffffLL, TYLO_ERR_UNSUPPORTED, "%s: n_splits*H*B too large", who);
  return TYLO_OK;
}

}  // namespace tylo

using namespace tylo;

extern "C" int32_t tylo_b200_decode_suggest_splits(int32_t Sk, int32_t Hkv, int32_t B) {
  if (Sk <= 0 || Hkv <= 0 || B <= 0) return 1;
  const int64_t groups = (int64_t)Hkv * B;
  // CTAs per SM by the size of the cache (keys x KV heads x batch; 512 bytes each at head dim 128), measured with
  // the one-launch form, back-to-back launches on rotating buffers:
  //   up to ~0.8 GB   one CTA per SM: start-up and the closing merge are paid once per SM and the merge stays narrow
  //                   (537 MB as 8 heads x 131,072 keys: 77-84 us against 83-85 with two per SM and 98 with eight;
  //                   as ONE head x 1,048,576 keys: 75-80 us with 148 splits against 94 with 296 and 183 with 1,184);
  //   up to ~3 GB     four per SM (1.07 GB: 162 us against 173 with one; 2.1 GB: 311 against 329);
  //   above           eight per SM: CTAs that finish early make room for the rest (4.3 GB: 602 us against 657).
  const int64_t key_heads = (int64_t)Sk * groups;
  const int per_sm = key_heads < 1536 * 1024 ? 1 : (key_heads < 6 * 1024 * 1024 ? 4 : 8);
  const int64_t target = (int64_t)sm_count() * per_sm;
  int64_t n = (target + groups - 1) / groups;
  const int64_t max_by_len = (Sk + 255) / 256;          // keep at least 256 keys per split
  if (n > max_by_len) n = max_by_len;
  if (n < 1) n = 1;
  return (int32_t)n;
}

extern "C" int32_t tylo_b200_decode_split(const void* Q, const void* K, const void* V, const int32_t* lengths,
                                          float* O_partial, float* M_partial, float* L_partial, int32_t n_splits,
                                          int32_t Dk, int32_t Dv, int32_t Sk, int32_t H, int32_t Hkv, int32_t B,
                                          int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(Q && K && V && lengths && O_partial && M_partial && L_partial, TYLO_ERR_INVALID_ARGUMENT,
               "decode_split: all pointers must be non-null");
  if (int32_t rc = check_decode_dims("decode_split", n_splits, Dk, Dv, Sk, H, Hkv, B)) return rc;
  TYLO_REQUIRE(aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O_partial), TYLO_ERR_MISALIGNED,
               "decode_split: pointers must be 16-byte aligned");
  const DecodeTail none{};
  const DecodePages dense{};
  TYLO_DISPATCH_DTYPE(dtype, T, return (decode_split_dispatch<T>(Q, K, V, lengths, O_partial, M_partial, L_partial,
                                                                 n_splits, Dk, Dv, Sk, H, Hkv, B, none, dense,
                                                                 (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_decode_combine(void* O, float* O_merged, float* M_merged, float* L_merged,
                                            const float* O_partial, const float* M_partial, const float* L_partial,
                                            int32_t n_splits, int64_t o_stride, int64_t ml_stride, int32_t Dv,
                                            int32_t H, int32_t B, int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(O_partial && M_partial && L_partial, TYLO_ERR_INVALID_ARGUMENT,
               "decode_combine: partial buffers must be non-null");
  TYLO_REQUIRE(O || O_merged, TYLO_ERR_INVALID_ARGUMENT, "decode_combine: no output requested");
  TYLO_REQUIRE((O_merged == nullptr) == (M_merged == nullptr) && (M_merged == nullptr) == (L_merged == nullptr),
               TYLO_ERR_INVALID_ARGUMENT, "decode_combine: O_merged, M_merged and L_merged go together");
  TYLO_REQUIRE(n_splits > 0 && Dv > 0 && H > 0 && B > 0, TYLO_ERR_INVALID_ARGUMENT,
               "decode_combine: extents must be positive");
  TYLO_REQUIRE(o_stride >= (int64_t)H * B * Dv || n_splits == 1, TYLO_ERR_INVALID_ARGUMENT,
               "decode_combine: o_stride (%lld) smaller than one partial (%lld)", (long long)o_stride,
               (long long)H * B * Dv);
  TYLO_REQUIRE(ml_stride >= (int64_t)H * B || n_splits == 1, TYLO_ERR_INVALID_ARGUMENT,
               "decode_combine: ml_stride (%lld) smaller than one partial (%lld)", (long long)ml_stride,
               (long long)H * B);
  TYLO_DISPATCH_DTYPE(dtype, T, return (decode_combine_dispatch<T>(O, O_merged, M_merged, L_merged, O_partial,
                                                                   M_partial, L_partial, n_splits, o_stride,
                                                                   ml_stride, Dv, H, B, (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_decode_attention(void* O, const void* Q, const void* K, const void* V,
                                              const int32_t* lengths, float* O_partial, float* M_partial,
                                              float* L_partial, int32_t n_splits, int32_t Dk, int32_t Dv, int32_t Sk,
                                              int32_t H, int32_t Hkv, int32_t B, int32_t dtype,
                                              tylo_stream_t stream) {
  TYLO_REQUIRE(O, TYLO_ERR_INVALID_ARGUMENT, "decode_attention: O must be non-null");
  TYLO_REQUIRE(aligned16(O), TYLO_ERR_MISALIGNED, "decode_attention: O must be 16-byte aligned");
  int32_t rc = tylo_b200_decode_split(Q, K, V, lengths, O_partial, M_partial, L_partial, n_splits, Dk, Dv, Sk, H,
                                      Hkv, B, dtype, stream);
  if (rc) return rc;
  return tylo_b200_decode_combine(O, nullptr, nullptr, nullptr, O_partial, M_partial, L_partial, n_splits,
                                  (int64_t)H * B * Dv, (int64_t)H * B, Dv, H, B, dtype, stream);
}

// ---- one launch: split, merge and (for a sharded sequence) the exchange between GPUs ------------------------
extern "C" int64_t tylo_b200_decode_ticket_count(int32_t n_splits, int32_t Hkv, int32_t B) {
  if (n_splits <= 0 || Hkv <= 0 || B <= 0) return 0;
  return (int64_t)Hkv * B * (decode_groups(n_splits) + 1);
}

static int32_t decode_one_launch(void* O, const void* Q, const void* K, const void* V, const int32_t* lengths,
                                 float* O_partial, float* M_partial, float* L_partial, int32_t* tickets,
                                 int32_t n_splits, const ExchangePeers* peers, int rank, int world, int32_t Dk,
                                 int32_t Dv, int32_t Sk, int32_t H, int32_t Hkv, int32_t B, int32_t dtype,
                                 int64_t timeout_us, tylo_stream_t stream, const DecodePages& pages = DecodePages{}) {
  DecodeTail tail{};
  tail.tickets = tickets; tail.O = O; tail.rank = rank; tail.world = world;
  if (peers) tail.peers = *peers;
  tail.timeout_ns = timeout_us > 0 ? (unsigned long long)timeout_us * 1000ull : 2000000000ull;   // default: two seconds
  TYLO_DISPATCH_DTYPE(dtype, T, return (decode_split_dispatch<T>(Q, K, V, lengths, O_partial, M_partial, L_partial,
                                                                 n_splits, Dk, Dv, Sk, H, Hkv, B, tail, pages,
                                                                 (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_decode_attention_fused(void* O, const void* Q, const void* K, const void* V,
                                                    const int32_t* lengths, float* O_partial, float* M_partial,
                                                    float* L_partial, int32_t* tickets, int32_t n_splits, int32_t Dk,
                                                    int32_t Dv, int32_t Sk, int32_t H, int32_t Hkv, int32_t B,
                                                    int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(O && Q && K && V && lengths && O_partial && M_partial && L_partial, TYLO_ERR_INVALID_ARGUMENT,
               "decode_attention_fused: all pointers must be non-null");
  if (int32_t rc = check_decode_dims("decode_attention_fused", n_splits, Dk, Dv, Sk, H, Hkv, B)) return rc;
  TYLO_REQUIRE(aligned16(O) && aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O_partial), TYLO_ERR_MISALIGNED,
               "decode_attention_fused: pointers must be 16-byte aligned");
  if (!tickets || !decode_mma_eligible(dtype, Dk, Dv, H, Hkv))    // shapes of the scalar kernel: two launches
    return tylo_b200_decode_attention(O, Q, K, V, lengths, O_partial, M_partial, L_partial, n_splits, Dk, Dv, Sk, H,
                                      Hkv, B, dtype, stream);
  return decode_one_launch(O, Q, K, V, lengths, O_partial, M_partial, L_partial, tickets, n_splits, nullptr, 0, 1, Dk,
                           Dv, Sk, H, Hkv, B, dtype, 0, stream);
}

extern "C" int32_t tylo_b200_decode_attention_paged(void* O, const void* Q, const void* K_pages, const void* V_pages,
                                                    const int32_t* block_table, const int32_t* lengths,
                                                    float* O_partial, float* M_partial, float* L_partial,
                                                    int32_t* tickets, int32_t n_splits, int32_t page_size,
                                                    int32_t max_pages, int32_t Dk, int32_t Dv, int32_t H, int32_t Hkv,
                                                    int32_t B, int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(O && Q && K_pages && V_pages && block_table && lengths && O_partial && M_partial && L_partial && tickets,
               TYLO_ERR_INVALID_ARGUMENT, "decode_attention_paged: all pointers must be non-null");
  TYLO_REQUIRE(page_size > 0 && max_pages > 0 && (int64_t)page_size * max_pages <= 0x7fffffffLL, TYLO_ERR_INVALID_ARGUMENT,
               "decode_attention_paged: page_size and max_pages must be positive");
  const int Sk = page_size * max_pages;          // longest sequence the table can describe
  if (int32_t rc = check_decode_dims("decode_attention_paged", n_splits, Dk, Dv, Sk, H, Hkv, B)) return rc;
  TYLO_REQUIRE(decode_mma_eligible(dtype, Dk, Dv, H, Hkv), TYLO_ERR_UNSUPPORTED,
               "decode_attention_paged: needs 16-bit storage, Dk == Dv in {64, 128} and at most 16 query heads per kv head");
  TYLO_REQUIRE(page_size % (Dk == 128 ? 16 : 32) == 0, TYLO_ERR_UNSUPPORTED,
               "decode_attention_paged: page_size (%d) must be a multiple of %d keys", page_size, Dk == 128 ? 16 : 32);
  TYLO_REQUIRE(aligned16(O) && aligned16(Q) && aligned16(K_pages) && aligned16(V_pages) && aligned16(O_partial),
               TYLO_ERR_MISALIGNED, "decode_attention_paged: pointers must be 16-byte aligned");
  DecodePages pages{block_table, page_size, max_pages};
  return decode_one_launch(O, Q, K_pages, V_pages, lengths, O_partial, M_partial, L_partial, tickets, n_splits, nullptr, 0, 1,
                           Dk, Dv, Sk, H, Hkv, B, dtype, 0, stream, pages);
}

extern "C" int32_t tylo_b200_decode_attention_sharded(void* O, const void* Q, const void* K, const void* V,
                                                      const int32_t* lengths_local, float* O_partial, float* M_partial,
                                                      float* L_partial, int32_t* tickets, int32_t n_splits,
                                                      void* const* peer_buffers, int32_t rank, int32_t world,
                                                      int32_t Dk, int32_t Dv, int32_t Sk_local, int32_t H, int32_t Hkv,
                                                      int32_t B, int32_t dtype, int64_t timeout_us,
                                                      tylo_stream_t stream) {
  TYLO_REQUIRE(O && Q && K && V && lengths_local && O_partial && M_partial && L_partial && peer_buffers,
               TYLO_ERR_INVALID_ARGUMENT, "decode_attention_sharded: all pointers must be non-null");
  if (int32_t rc = check_decode_dims("decode_attention_sharded", n_splits, Dk, Dv, Sk_local, H, Hkv, B)) return rc;
  TYLO_REQUIRE(world >= 1 && world <= kMaxExchangeWorld, TYLO_ERR_UNSUPPORTED,
               "decode_attention_sharded: world size %d outside 1..%d", world, kMaxExchangeWorld);
  TYLO_REQUIRE(rank >= 0 && rank < world, TYLO_ERR_INVALID_ARGUMENT, "decode_attention_sharded: rank %d outside 0..%d",
               rank, world - 1);
  TYLO_REQUIRE(aligned16(O) && aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(O_partial), TYLO_ERR_MISALIGNED,
               "decode_attention_sharded: pointers must be 16-byte aligned");
  if (!tickets || !decode_mma_eligible(dtype, Dk, Dv, H, Hkv)) {
    // two launches: the split kernel, then the exchange kernel
    if (int32_t rc = tylo_b200_decode_split(Q, K, V, lengths_local, O_partial, M_partial, L_partial, n_splits, Dk, Dv,
                                            Sk_local, H, Hkv, B, dtype, stream))
      return rc;
    return tylo_b200_decode_exchange(O, O_partial, M_partial, L_partial, n_splits, (int64_t)H * B * Dv, (int64_t)H * B,
                                     peer_buffers, rank, world, Dv, H, B, dtype, timeout_us, stream);
  }
  ExchangePeers peers{};
  for (int r = 0; r < world; ++r) {
    TYLO_REQUIRE(peer_buffers[r] && aligned16(peer_buffers[r]), TYLO_ERR_INVALID_ARGUMENT,
                 "decode_attention_sharded: peer buffer %d is null or not 16-byte aligned", r);
    peers.buf[r] = static_cast<float*>(peer_buffers[r]);
  }
  return decode_one_launch(O, Q, K, V, lengths_local, O_partial, M_partial, L_partial, tickets, n_splits, &peers, rank,
                           world, Dk, Dv, Sk_local, H, Hkv, B, dtype, timeout_us, stream);
}

// ---- decode without caller-provided scratch ------------------------------------------------------------
// Some hosts cannot hand the library a scratch buffer: code running where cudaMalloc is off limits —
// a serving loop that has frozen its memory pool, a plugin called from a runtime that owns every
// byte of device memory, a callback with no allocator in reach.  For them the split partials live in
// a fixed array that is part of the library image on every GPU that loads it.
//
// The array's name is only a host-side handle: its device address is looked up once per device with
// cudaGetSymbolAddress (while that device is current) and that address is what the kernels receive.
namespace tylo {

constexpr size_t kStaticScratchFloats = size_t(2) << 20;   // 8 MiB of fp32, held from load until exit
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
static float* g_static_scratch_addr[kMaxDevices] = {};

// First call on a device resolves the address (no allocation); later calls reuse it.
static int32_t static_scratch_for_current_device(float** out) {
  int dev = -1;
  TYLO_CUDA_OK(cudaGetDevice(&dev));
  TYLO_REQUIRE(dev >= 0 && dev < kMaxDevices, TYLO_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  float* p = __atomic_load_n(&g_static_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    TYLO_CUDA_OK(cudaGetSymbolAddress(&sym, g_decode_static_scratch));
    TYLO_REQUIRE(sym != nullptr, TYLO_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    p = static_cast<float*>(sym);
    __atomic_store_n(&g_static_scratch_addr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return TYLO_OK;
}

}  // namespace tylo

extern "C" int64_t tylo_b200_decode_static_scratch_floats(void) { return (int64_t)tylo::kStaticScratchFloats; }

extern "C" int32_t tylo_b200_decode_attention_static(void* O, const void* Q, const void* K, const void* V,
                                                     const int32_t* lengths, int32_t n_splits, int32_t Dk,
                                                     int32_t Dv, int32_t Sk, int32_t H, int32_t Hkv, int32_t B,
                                                     int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(O, TYLO_ERR_INVALID_ARGUMENT, "decode_attention_static: O must be non-null");
  if (int32_t rc = check_decode_dims("decode_attention_static", n_splits, Dk, Dv, Sk, H, Hkv, B)) return rc;
  const int64_t need = (int64_t)n_splits * B * H * ((int64_t)Dv + 2);
  TYLO_REQUIRE(need <= (int64_t)kStaticScratchFloats, TYLO_ERR_WORKSPACE,
               "decode_attention_static: n_splits*B*H*(Dv+2) = %lld floats exceeds the built-in scratch of %lld "
               "floats; lower n_splits or use tylo_b200_decode_attention with your own scratch",
               (long long)need, (long long)kStaticScratchFloats);
  float* base = nullptr;
  if (int32_t rc = static_scratch_for_current_device(&base)) return rc;
  // every (split, batch, head) slot is overwritten by the split kernel, so nothing has to be cleared
  const size_t n_o = (size_t)n_splits * B * H * Dv, n_ml = (size_t)n_splits * B * H;
  float* o_part = base;
  float* m_part = base + n_o;
  float* l_part = m_part + n_ml;
  return tylo_b200_decode_attention(O, Q, K, V, lengths, o_part, m_part, l_part, n_splits, Dk, Dv, Sk, H, Hkv, B,
                                    dtype, stream);
}
