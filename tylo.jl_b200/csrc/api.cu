// C-ABI entry points for the attention family plus the library-wide status plumbing.
// Argument checks mirror the @assert lines of the Julia wrappers they stand in for
// (attention.jl:234-237,318-326; flex.jl:325-334,466-476) and run before anything is enqueued.
#include <cmath>
#include <cstring>

#include "attn_dispatch.cuh"

namespace tylo {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static int32_t check_attn_dims(const char* who, int Dk, int Dv, int Sq, int Sk, int H, int Hkv, int B) {
  TYLO_REQUIRE(Dk > 0 && Dv > 0 && Sq > 0 && Sk > 0 && H > 0 && Hkv > 0 && B > 0, TYLO_ERR_INVALID_ARGUMENT,
               "%s: extents must be positive (Dk=%d Dv=%d Sq=%d Sk=%d H=%d Hkv=%d B=%d)", who, Dk, Dv, Sq, Sk, H,
               Hkv, B);
  TYLO_REQUIRE(H % Hkv == 0, TYLO_ERR_INVALID_ARGUMENT, "%s: Heads (%d) must be a multiple of Heads_KV (%d)", who,
               H, Hkv);
  return TYLO_OK;
}

static int32_t fill_mods(const char* who, AttnParams& p, const tylo_mask_desc* mask, const tylo_score_desc* score) {
  p.mask_flags = 0; p.window = 0; p.prefix_len = 0; p.doc_q = nullptr; p.doc_kv = nullptr; p.doc_stride = 0;
  p.score_flags = 0; p.cap = 1.f; p.slopes = nullptr; p.d_slopes = nullptr;
  p.bias = nullptr; p.d_bias = nullptr; p.bias_heads = 1; p.bias_batch = 1;
  p.n_or = 0;
  int n_clauses = 0;
  for (const tylo_mask_desc* m = mask; m; m = m->or_next, ++n_clauses) {
    TYLO_REQUIRE(n_clauses <= kMaxOrClauses, TYLO_ERR_UNSUPPORTED, "%s: more than %d OR-ed mask clauses", who,
                 kMaxOrClauses + 1);
    const uint32_t known = TYLO_MASK_CAUSAL | TYLO_MASK_SLIDING | TYLO_MASK_DOCUMENT | TYLO_MASK_PREFIX |
                           TYLO_MASK_PREFIX_LM;
    TYLO_REQUIRE((m->flags & ~known) == 0, TYLO_ERR_UNSUPPORTED, "%s: unknown mask flags 0x%x", who, m->flags);
    MaskClause c{m->flags, m->window, m->prefix_len, nullptr, nullptr, 0};
    if (m->flags & TYLO_MASK_SLIDING)
      TYLO_REQUIRE(m->window >= 0, TYLO_ERR_INVALID_ARGUMENT, "%s: sliding window must be >= 0", who);
    if (m->flags & TYLO_MASK_DOCUMENT) {
      TYLO_REQUIRE(m->doc_q && m->doc_kv, TYLO_ERR_INVALID_ARGUMENT, "%s: DocumentMask needs doc_q and doc_kv", who);
      TYLO_REQUIRE(m->doc_q_len >= (int64_t)p.input_pos + p.Sq && p.input_pos >= 0, TYLO_ERR_INVALID_ARGUMENT,
                   "%s: doc_q holds %lld ids but query positions reach %lld", who, (long long)m->doc_q_len,
                   (long long)p.input_pos + p.Sq);
      TYLO_REQUIRE(m->doc_kv_len >= p.Sk, TYLO_ERR_INVALID_ARGUMENT,
                   "%s: doc_kv holds %lld ids but there are %d keys", who, (long long)m->doc_kv_len, p.Sk);
      TYLO_REQUIRE(m->doc_batch_stride >= 0, TYLO_ERR_INVALID_ARGUMENT, "%s: negative doc_batch_stride", who);
      c.doc_q = m->doc_q; c.doc_kv = m->doc_kv; c.doc_stride = m->doc_batch_stride;
    }
    if (n_clauses == 0) {
      p.mask_flags = c.flags; p.window = c.window; p.prefix_len = c.prefix_len;
      p.doc_q = c.doc_q; p.doc_kv = c.doc_kv; p.doc_stride = c.doc_stride;
    } else {
      p.or_clause[p.n_or++] = c;
    }
  }
  if (score) {
    const uint32_t known = TYLO_SCORE_ALIBI | TYLO_SCORE_SOFTCAP | TYLO_SCORE_SOFTCAP_FIRST | TYLO_SCORE_BIAS;
    TYLO_REQUIRE((score->flags & ~known) == 0, TYLO_ERR_UNSUPPORTED, "%s: unknown score flags 0x%x", who,
                 score->flags);
    p.score_flags = score->flags;
    if (score->flags & TYLO_SCORE_SOFTCAP) {
      TYLO_REQUIRE(score->cap > 0.f && std::isfinite(score->cap), TYLO_ERR_INVALID_ARGUMENT,
                   "%s: soft cap must be positive and finite", who);
      p.cap = score->cap;
    }
    if (score->flags & TYLO_SCORE_ALIBI) {
      TYLO_REQUIRE(score->slopes, TYLO_ERR_INVALID_ARGUMENT, "%s: AliBiScore needs slopes", who);
      p.slopes = score->slopes; p.d_slopes = score->d_slopes;
    }
    if (score->flags & TYLO_SCORE_BIAS) {
      TYLO_REQUIRE(score->bias, TYLO_ERR_INVALID_ARGUMENT, "%s: BiasScore needs a bias table", who);
      TYLO_REQUIRE(score->bias_heads > 0 && score->bias_batch > 0, TYLO_ERR_INVALID_ARGUMENT,
                   "%s: BiasScore extents must be positive (heads %d, batch %d)", who, score->bias_heads,
                   score->bias_batch);
      // the kernels read table rows with 16-byte loads and add to the gradient with 16-byte reductions
      TYLO_REQUIRE(aligned16(score->bias) && aligned16(score->d_bias), TYLO_ERR_MISALIGNED,
                   "%s: the bias table and its gradient must be 16-byte aligned", who);
      p.bias = score->bias; p.d_bias = score->d_bias; p.bias_heads = score->bias_heads; p.bias_batch = score->bias_batch;
    }
  }
  return TYLO_OK;
}

// Host-built block list (mods.jl:436-476): the analytic block range is not used with it.
static int32_t fill_block_mask(const char* who, AttnParams& p, const int32_t* count, const int32_t* idx,
                               const int32_t* full, int32_t stride, int32_t tile_m, int32_t tile_n) {
  TYLO_REQUIRE(count && idx && full, TYLO_ERR_INVALID_ARGUMENT, "%s: count, idx and full must be non-null", who);
  TYLO_REQUIRE(tile_m > 0 && tile_n > 0 && tile_m % 32 == 0 && tile_n % 32 == 0, TYLO_ERR_UNSUPPORTED,
               "%s: block edges must be positive multiples of 32 (TILE_M=%d, TILE_N=%d)", who, tile_m, tile_n);
  TYLO_REQUIRE(stride > 0, TYLO_ERR_INVALID_ARGUMENT, "%s: bm_stride must be positive", who);
  p.bm_count = count; p.bm_idx = idx; p.bm_full = full;
  p.bm_stride = stride; p.bm_tm = tile_m; p.bm_tn = tile_n;
  p.block_sparse = 0;
  return TYLO_OK;
}

static void fill_dims(AttnParams& p, int Dk, int Dv, int Sq, int Sk, int H, int Hkv, int B, int input_pos) {
  std::memset(&p, 0, sizeof(p));
  p.Dk = Dk; p.Dv = Dv; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv; p.B = B; p.G = H / Hkv;
  p.input_pos = input_pos;
}

}  // namespace tylo

using namespace tylo;

extern "C" int32_t tylo_b200_version(void) { return TYLO_B200_VERSION; }

extern "C" const char* tylo_b200_last_error(void) { return g_err; }

extern "C" int32_t tylo_b200_device_status(int32_t* code) {
  TYLO_REQUIRE(code, TYLO_ERR_INVALID_ARGUMENT, "device_status: code must be non-null");
  TYLO_CUDA_OK(cudaDeviceSynchronize());
  int v = 0;
  if (int32_t rc = attn_fwd_sm100_status(&v)) return rc;
  if (v == 0) {
    int w = 0;
    if (int32_t rc = attn_bwd_sm100_status(&w)) return rc;
    if (w != 0) v = 1000 + w;   // backward kernels report 1000 + their own code
  }
  *code = v;
  TYLO_REQUIRE(v == 0, TYLO_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (code %d)", v);
  return TYLO_OK;
}

extern "C" const char* tylo_b200_status_string(int32_t status) {
  switch (status) {
    case TYLO_OK: return "ok";
    case TYLO_ERR_INVALID_ARGUMENT: return "invalid argument";
    case TYLO_ERR_UNSUPPORTED: return "unsupported by libtylo_b200";
    case TYLO_ERR_MISALIGNED: return "pointer not 16-byte aligned";
    case TYLO_ERR_CUDA: return "CUDA error";
    case TYLO_ERR_NCCL: return "NCCL error";
    case TYLO_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case TYLO_ERR_WORKSPACE: return "workspace too small";
    default: return "unknown status";
  }
}

extern "C" int32_t tylo_b200_attention_fwd(void* O, const void* Q, const void* K, const void* V, float* M, float* L,
                                           const int32_t* k_lengths, const int32_t* q_lengths, int32_t Dk,
                                           int32_t Dv, int32_t Sq, int32_t Sk, int32_t H, int32_t Hkv, int32_t B,
                                           int32_t input_pos, int32_t causal, int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(O && Q && K && V, TYLO_ERR_INVALID_ARGUMENT, "attention_fwd: O, Q, K and V must be non-null");
  if (int32_t rc = check_attn_dims("attention_fwd", Dk, Dv, Sq, Sk, H, Hkv, B)) return rc;
  TYLO_REQUIRE(aligned16(O) && aligned16(Q) && aligned16(K) && aligned16(V), TYLO_ERR_MISALIGNED,
               "attention_fwd: pointers must be 16-byte aligned");
  AttnParams p;
  fill_dims(p, Dk, Dv, Sq, Sk, H, Hkv, B, input_pos);
  p.scale = 1.0f / std::sqrt((float)Dk);             // attention.jl:240
  p.mask_flags = causal ? TYLO_MASK_CAUSAL : 0u;
  p.k_lengths = k_lengths; p.q_lengths = q_lengths;
  p.natural_stats = 0; p.block_sparse = 1; p.cap = 1.f;
  return attn_fwd_dispatch(O, Q, K, V, M, L, p, dtype, (cudaStream_t)stream);
}

extern "C" int64_t tylo_b200_attention_bwd_workspace_bytes(int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                                           int32_t H, int32_t Hkv, int32_t B, int32_t dtype) {
  return attn_bwd_workspace_bytes(Dk, Dv, Sq, Sk, H, Hkv, B, dtype);
}

static int32_t bwd_common(const char* who, void* dQ, void* dK, void* dV, const void* Q, const void* K,
                          const void* V, const void* O, const void* dO, const float* M, const float* L,
                          float* Delta, void* workspace, int64_t workspace_bytes, AttnParams& p, int32_t dtype,
                          tylo_stream_t stream) {
  TYLO_REQUIRE(dQ && dK && dV && Q && K && V && O && dO, TYLO_ERR_INVALID_ARGUMENT,
               "%s: gradient, input and output arrays must be non-null", who);
  TYLO_REQUIRE(M && L, TYLO_ERR_INVALID_ARGUMENT, "%s: checkpoints M and L from the forward are required", who);
  TYLO_REQUIRE(Delta, TYLO_ERR_INVALID_ARGUMENT, "%s: scratch Delta is required", who);
  TYLO_REQUIRE(aligned16(dQ) && aligned16(dK) && aligned16(dV) && aligned16(Q) && aligned16(K) && aligned16(V) &&
                   aligned16(O) && aligned16(dO), TYLO_ERR_MISALIGNED, "%s: pointers must be 16-byte aligned", who);
  const int64_t need = attn_bwd_workspace_bytes(p.Dk, p.Dv, p.Sq, p.Sk, p.H, p.Hkv, p.B, dtype);
  TYLO_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), TYLO_ERR_WORKSPACE,
               "%s: workspace of %lld bytes required, %lld given", who, (long long)need,
               (long long)(workspace ? workspace_bytes : 0));
  return attn_bwd_dispatch(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, workspace, p, dtype, (cudaStream_t)stream);
}

extern "C" int32_t tylo_b200_attention_bwd(void* dQ, void* dK, void* dV, const void* Q, const void* K,
                                           const void* V, const void* O, const void* dO, const float* M,
                                           const float* L, void* dO_scaled, float* Delta, void* workspace,
                                           int64_t workspace_bytes, const int32_t* k_lengths,
                                           const int32_t* q_lengths, int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                           int32_t H, int32_t Hkv, int32_t B, int32_t input_pos, int32_t causal,
                                           int32_t dtype, tylo_stream_t stream) {
  (void)dO_scaled;
  if (int32_t rc = check_attn_dims("attention_bwd", Dk, Dv, Sq, Sk, H, Hkv, B)) return rc;
  AttnParams p;
  fill_dims(p, Dk, Dv, Sq, Sk, H, Hkv, B, input_pos);
  p.scale = 1.0f / std::sqrt((float)Dk);
  p.mask_flags = causal ? TYLO_MASK_CAUSAL : 0u;
  p.k_lengths = k_lengths; p.q_lengths = q_lengths;
  p.natural_stats = 0; p.block_sparse = 1; p.cap = 1.f;
  return bwd_common("attention_bwd", dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, workspace, workspace_bytes, p, dtype,
                    stream);
}

extern "C" int32_t tylo_b200_flex_attention_fwd(void* O, const void* Q, const void* K, const void* V, float* M,
                                                float* L, const tylo_mask_desc* mask, const tylo_score_desc* score,
                                                int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk, int32_t H,
                                                int32_t Hkv, int32_t B, int32_t input_pos, float qk_scale,
                                                int32_t block_sparse, int32_t dtype, tylo_stream_t stream) {
  TYLO_REQUIRE(O && Q && K && V, TYLO_ERR_INVALID_ARGUMENT, "flex_attention_fwd: O, Q, K and V must be non-null");
  if (int32_t rc = check_attn_dims("flex_attention_fwd", Dk, Dv, Sq, Sk, H, Hkv, B)) return rc;
  TYLO_REQUIRE(aligned16(O) && aligned16(Q) && aligned16(K) && aligned16(V), TYLO_ERR_MISALIGNED,
               "flex_attention_fwd: pointers must be 16-byte aligned");
  AttnParams p;
  fill_dims(p, Dk, Dv, Sq, Sk, H, Hkv, B, input_pos);
  if (int32_t rc = fill_mods("flex_attention_fwd", p, mask, score)) return rc;
  p.scale = qk_scale > 0.f ? qk_scale : 1.0f / std::sqrt((float)Dk);  // flex.jl:337
  p.natural_stats = 1; p.block_sparse = block_sparse ? 1 : 0;
  return attn_fwd_dispatch(O, Q, K, V, M, L, p, dtype, (cudaStream_t)stream);
}

extern "C" int32_t tylo_b200_flex_attention_fwd_block_mask(
    void* O, const void* Q, const void* K, const void* V, float* M, float* L, const tylo_mask_desc* mask,
    const tylo_score_desc* score, const int32_t* bm_count, const int32_t* bm_idx, const int32_t* bm_full,
    int32_t bm_stride, int32_t tile_m, int32_t tile_n, int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk, int32_t H,
    int32_t Hkv, int32_t B, int32_t input_pos, float qk_scale, int32_t dtype, tylo_stream_t stream) {
  const char* who = "flex_attention_fwd_block_mask";
  TYLO_REQUIRE(O && Q && K && V, TYLO_ERR_INVALID_ARGUMENT, "%s: O, Q, K and V must be non-null", who);
  if (int32_t rc = check_attn_dims(who, Dk, Dv, Sq, Sk, H, Hkv, B)) return rc;
  TYLO_REQUIRE(aligned16(O) && aligned16(Q) && aligned16(K) && aligned16(V), TYLO_ERR_MISALIGNED,
               "%s: pointers must be 16-byte aligned", who);
  AttnParams p;
  fill_dims(p, Dk, Dv, Sq, Sk, H, Hkv, B, input_pos);
  if (int32_t rc = fill_mods(who, p, mask, score)) return rc;
  if (int32_t rc = fill_block_mask(who, p, bm_count, bm_idx, bm_full, bm_stride, tile_m, tile_n)) return rc;
  p.scale = qk_scale > 0.f ? qk_scale : 1.0f / std::sqrt((float)Dk);  // flex.jl:337
  p.natural_stats = 1;
  return attn_fwd_dispatch(O, Q, K, V, M, L, p, dtype, (cudaStream_t)stream);
}

extern "C" int32_t tylo_b200_flex_attention_bwd_block_mask(
    void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V, const void* O, const void* dO,
    const float* M, const float* L, float* Delta, void* workspace, int64_t workspace_bytes,
    const tylo_mask_desc* mask, const tylo_score_desc* score, const int32_t* bm_count, const int32_t* bm_idx,
    const int32_t* bm_full, int32_t bm_stride, int32_t tile_m, int32_t tile_n, int32_t Dk, int32_t Dv, int32_t Sq,
    int32_t Sk, int32_t H, int32_t Hkv, int32_t B, int32_t input_pos, float qk_scale, int32_t dtype,
    tylo_stream_t stream) {
  const char* who = "flex_attention_bwd_block_mask";
  if (int32_t rc = check_attn_dims(who, Dk, Dv, Sq, Sk, H, Hkv, B)) return rc;
  AttnParams p;
  fill_dims(p, Dk, Dv, Sq, Sk, H, Hkv, B, input_pos);
  if (int32_t rc = fill_mods(who, p, mask, score)) return rc;
  if (int32_t rc = fill_block_mask(who, p, bm_count, bm_idx, bm_full, bm_stride, tile_m, tile_n)) return rc;
  p.scale = qk_scale > 0.f ? qk_scale : 1.0f / std::sqrt((float)Dk);
  p.natural_stats = 1;
  return bwd_common(who, dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, workspace, workspace_bytes, p, dtype, stream);
}

extern "C" int32_t tylo_b200_flex_attention_bwd(void* dQ, void* dK, void* dV, const void* Q, const void* K,
                                                const void* V, const void* O, const void* dO, const float* M,
                                                const float* L, void* dO_scaled, float* Delta, void* workspace,
                                                int64_t workspace_bytes, const tylo_mask_desc* mask,
                                                const tylo_score_desc* score, int32_t Dk, int32_t Dv, int32_t Sq,
                                                int32_t Sk, int32_t H, int32_t Hkv, int32_t B, int32_t input_pos,
                                                float qk_scale, int32_t block_sparse, int32_t dtype,
                                                tylo_stream_t stream) {
  (void)dO_scaled;
  if (int32_t rc = check_attn_dims("flex_attention_bwd", Dk, Dv, Sq, Sk, H, Hkv, B)) return rc;
  AttnParams p;
  fill_dims(p, Dk, Dv, Sq, Sk, H, Hkv, B, input_pos);
  if (int32_t rc = fill_mods("flex_attention_bwd", p, mask, score)) return rc;
  p.scale = qk_scale > 0.f ? qk_scale : 1.0f / std::sqrt((float)Dk);
  p.natural_stats = 1; p.block_sparse = block_sparse ? 1 : 0;
  return bwd_common("flex_attention_bwd", dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, workspace, workspace_bytes, p,
                    dtype, stream);
}
