// Parameters shared by every attention kernel, and the element-wise score/mask mods
// (device restatement of the mod bodies in src/attention/mods.jl).
#pragma once
#include "common.cuh"

namespace tylo {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// One conjunction of mask terms; a mask is clause 0 (the AttnParams fields) OR-ed with `or_clause`s.
struct MaskClause {
  uint32_t flags;
  int window, prefix_len;
  const int32_t* doc_q;
  const int32_t* doc_kv;
  long long doc_stride;
};
constexpr int kMaxOrClauses = 3;

struct AttnParams {
  int Dk, Dv, Sq, Sk, H, Hkv, B, G;
  int input_pos;
  float scale;            // qk scale applied to the raw dot product
  uint32_t mask_flags;    // TYLO_MASK_*
  int window, prefix_len;
  const int32_t* doc_q;
  const int32_t* doc_kv;
  long long doc_stride;   // per-batch stride of the id tables (0 = shared)
  uint32_t score_flags;   // TYLO_SCORE_*
  float cap;
  const float* slopes;
  float* d_slopes;
  const float* bias;      // (Sk, Sq, bias_heads, bias_batch) fp32, local row indices
  float* d_bias;
  int bias_heads, bias_batch;
  const int32_t* k_lengths;
  const int32_t* q_lengths;
  int natural_stats;      // 1: M/L in natural units (flex), 0: log2 units (attention!)
  int block_sparse;
  // Host-built coarse block mask (mods.jl:436-476), forward only: per query block of bm_tm rows the
  // list of key blocks (bm_tn keys each) to visit and whether mask_mod may be skipped there.
  const int32_t* bm_count;   // [n_qb]
  const int32_t* bm_idx;     // [n_qb][bm_stride], 0-based key block ids
  const int32_t* bm_full;    // [n_qb][bm_stride], != 0: fully unmasked
  int bm_tm, bm_tn, bm_stride;
  // OrMask (mods.jl:164-167) in disjunctive normal form: further clauses OR-ed with the mask above
  // (fp32-arithmetic kernels only; the analytic block range is not used with them).
  int n_or;
  MaskClause or_clause[kMaxOrClauses];
};

// Mask for one (q, kv) pair of absolute 0-based positions (mods.jl:101-167).
__device__ __forceinline__ bool clause_keep(uint32_t flags, int window, int prefix_len, const int32_t* doc_q,
                                            const int32_t* doc_kv, long long doc_stride, int b, int q, int kv) {
  bool keep = true;
  if (flags & TYLO_MASK_CAUSAL) keep = keep && (q >= kv);
  if (flags & TYLO_MASK_SLIDING) keep = keep && (q >= kv) && (q <= kv + window);
  if (flags & TYLO_MASK_PREFIX) keep = keep && (kv < prefix_len);
  if (flags & TYLO_MASK_PREFIX_LM) keep = keep && ((q >= kv) || (kv < prefix_len));
  if (flags & TYLO_MASK_DOCUMENT)
    keep = keep && (doc_q[(size_t)b * doc_stride + q] == doc_kv[(size_t)b * doc_stride + kv]);
  return keep;
}
__device__ __forceinline__ bool mask_keep(const AttnParams& p, int b, int q, int kv) {
  bool keep = clause_keep(p.mask_flags, p.window, p.prefix_len, p.doc_q, p.doc_kv, p.doc_stride, b, q, kv);
  for (int i = 0; i < p.n_or; ++i) {
    const MaskClause& c = p.or_clause[i];
    keep = keep || clause_keep(c.flags, c.window, c.prefix_len, c.doc_q, c.doc_kv, c.doc_stride, b, q, kv);
  }
  return keep;
}

// Additive part of the score-mod chain for one pair: ALiBi's slope * (q - kv) on absolute positions plus
// BiasScore's table entry on LOCAL row indices, heads and batch broadcast by modulo (mods.jl:205-237).
__device__ __forceinline__ size_t bias_index(const AttnParams& p, int b, int h, int row, int kv) {
  return (((size_t)(b % p.bias_batch) * p.bias_heads + (h % p.bias_heads)) * p.Sq + row) * p.Sk + kv;
}
__device__ __forceinline__ float score_additive(const AttnParams& p, float slope, int b, int h, int row, int qpos,
                                                int kv) {
  float add = 0.f;
  if (p.score_flags & TYLO_SCORE_ALIBI) add = slope * (float)(qpos - kv);
  if (p.score_flags & TYLO_SCORE_BIAS) add += p.bias[bias_index(p, b, h, row, kv)];
  return add;
}

// Score mod chain on the scaled score s0 (mods.jl:188-249); `add` = score_additive.  Returns the modded score.
__device__ __forceinline__ float score_apply(const AttnParams& p, float s0, float add) {
  float s = s0;
  const bool additive = p.score_flags & (TYLO_SCORE_ALIBI | TYLO_SCORE_BIAS), cap = p.score_flags & TYLO_SCORE_SOFTCAP;
  const bool cap_first = p.score_flags & TYLO_SCORE_SOFTCAP_FIRST;
  if (cap && cap_first) s = p.cap * tanhf(s / p.cap);
  if (additive) s += add;
  if (cap && !cap_first) s = p.cap * tanhf(s / p.cap);
  return s;
}

// VJP of the chain at the pre-mod score (mods.jl:288-319): given ds at the output, returns ds0 and,
// through ds_at_add, the gradient at the additive mods (times (q - kv) it sums to the ALiBi slope
// gradient; as it stands it is the bias gradient of the pair).
__device__ __forceinline__ float score_vjp(const AttnParams& p, float s0, float add, float ds, float* ds_at_add) {
  const bool additive = p.score_flags & (TYLO_SCORE_ALIBI | TYLO_SCORE_BIAS), cap = p.score_flags & TYLO_SCORE_SOFTCAP;
  const bool cap_first = p.score_flags & TYLO_SCORE_SOFTCAP_FIRST;
  float g = ds;
  if (cap && !cap_first) {  // softcap is the outer mod: its input is s0 (+ additive mods)
    const float in = additive ? s0 + add : s0;
    const float th = tanhf(in / p.cap);
    g *= (1.f - th * th);
  }
  *ds_at_add = g;           // additive mods pass the gradient through
  if (cap && cap_first) {
    const float th = tanhf(s0 / p.cap);
    g *= (1.f - th * th);
  }
  return g;
}

// Range of key positions [lo, hi) that can hold an unmasked pair for queries [q_lo, q_hi]
// (absolute positions): the analytic block lattice of mods.jl:345-413 reduced to the affine masks.
__device__ __forceinline__ void kv_range(const AttnParams& p, int q_lo, int q_hi, int k_len, int* lo, int* hi) {
  int l = 0, h = k_len;
  if (p.block_sparse && p.n_or == 0) {
    if (p.mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) h = min(h, q_hi + 1);
    if (p.mask_flags & TYLO_MASK_SLIDING) l = max(l, q_lo - p.window);
    if (p.mask_flags & TYLO_MASK_PREFIX) h = min(h, p.prefix_len);
  }
  if (h < l) h = l;
  *lo = l; *hi = h;
}

// Query range [lo, hi) (row indices, not positions) that can see keys [kv_lo, kv_hi].
__device__ __forceinline__ void q_range(const AttnParams& p, int kv_lo, int kv_hi, int q_len, int* lo, int* hi) {
  int l = 0, h = q_len;
  if (p.block_sparse && p.n_or == 0) {
    if (p.mask_flags & (TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING)) l = max(l, kv_lo - p.input_pos);
    if (p.mask_flags & TYLO_MASK_SLIDING) h = min(h, kv_hi + p.window - p.input_pos + 1);
  }
  if (h < l) h = l;
  *lo = l; *hi = h;
}

}  // namespace tylo
