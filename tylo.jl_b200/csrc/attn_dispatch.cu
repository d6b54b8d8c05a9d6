// Chooses, per call, between the tcgen05 kernels and the generic fp32-arithmetic kernels.
// There is no CPU path: a request no kernel covers returns TYLO_ERR_UNSUPPORTED.
#include "attn_dispatch.cuh"

namespace tylo {

// What the tensor-core kernels leave to the fp32-arithmetic kernels.  Forward: host-built block lists, and
// OR-ed mask clauses that hold a document term (the tensor-core forward reduces every clause to one interval of
// keys per row).  Backward: those, every OR-ed mask and bias tables (their gradient is accumulated with atomics
// there).
static bool or_with_documents(const AttnParams& p) {
  if (p.n_or == 0) return false;
  bool doc = (p.mask_flags & TYLO_MASK_DOCUMENT) != 0;
  for (int i = 0; i < p.n_or; ++i) doc = doc || (p.or_clause[i].flags & TYLO_MASK_DOCUMENT) != 0;
  return doc;
}
static bool fwd_needs_generic(const AttnParams& p) { return or_with_documents(p); }
static bool table_mods(const AttnParams& p) { return p.bm_count != nullptr || or_with_documents(p); }

int32_t attn_fwd_dispatch(void* O, const void* Q, const void* K, const void* V, float* M, float* L,
                          const AttnParams& p, int32_t dtype, cudaStream_t st) {
  if (!fwd_needs_generic(p) && attn_fwd_sm100_supported(p, dtype)) return attn_fwd_sm100(O, Q, K, V, M, L, p, dtype, st);
  if (dtype == TYLO_F32_TF32) dtype = TYLO_F32;      // no tensor-core form for this call: true fp32
  TYLO_DISPATCH_DTYPE(dtype, T, return attn_fwd_generic<T>(O, Q, K, V, M, L, p, st));
  return TYLO_OK;
}

// The workspace is sized for the tensor-core path whenever the dtype and head dim could take it
// (whether a given call does also depends on its optional arguments).
int64_t attn_bwd_workspace_bytes(int Dk, int Dv, int Sq, int, int H, int, int B, int32_t dtype) {
  if ((dtype == TYLO_BF16 || dtype == TYLO_F16) && Dk == Dv && Dk >= 8 && Dk % 8 == 0 && Dk <= 128)
    return attn_bwd_sm100_workspace_bytes(Sq, H, B);
  return 0;
}

int32_t attn_bwd_dispatch(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V,
                          const void* O, const void* dO, const float* M, const float* L, float* Delta,
                          void* workspace, const AttnParams& p, int32_t dtype, cudaStream_t st) {
  if (!table_mods(p) && attn_bwd_sm100_supported(p, dtype))
    return attn_bwd_sm100(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, workspace, p, dtype, st);
  TYLO_DISPATCH_DTYPE(dtype, T, return attn_bwd_generic<T>(dQ, dK, dV, Q, K, V, O, dO, M, L, Delta, p, st));
  return TYLO_OK;
}

}  // namespace tylo
