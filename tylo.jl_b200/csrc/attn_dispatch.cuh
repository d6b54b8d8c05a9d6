// Routing of the attention entry points to the kernels that implement them.
#pragma once
#include "attn_params.cuh"

namespace tylo {

// fp32-arithmetic kernels for any dtype / shape / mod (attn_generic.cu)
template <typename T>
int32_t attn_fwd_generic(void* O, const void* Q, const void* K, const void* V, float* M, float* L,
                         const AttnParams& p, cudaStream_t st);
template <typename T>
int32_t attn_bwd_generic(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V,
                         const void* O, const void* dO, const float* M, const float* L, float* Delta,
                         const AttnParams& p, cudaStream_t st);

// tcgen05 / TMEM / TMA forward for 16-bit storage (attn_fwd_sm100.cu).  `supported` tells whether
// the kernel covers this problem; the launch returns a status.
bool attn_fwd_sm100_supported(const AttnParams& p, int32_t dtype);
int32_t attn_fwd_sm100(void* O, const void* Q, const void* K, const void* V, float* M, float* L,
                       const AttnParams& p, int32_t dtype, cudaStream_t st);

// tcgen05 / TMEM / TMA backward for 16-bit storage (attn_bwd_sm100.cu); `workspace` holds one fp32
// per (query, head, batch): the log2-domain log-sum-exp derived from the saved (M, L).
bool attn_bwd_sm100_supported(const AttnParams& p, int32_t dtype);
int64_t attn_bwd_sm100_workspace_bytes(int Sq, int H, int B);
int32_t attn_bwd_sm100(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V, const void* O,
                       const void* dO, const float* M, const float* L, float* Delta, void* workspace,
                       const AttnParams& p, int32_t dtype, cudaStream_t st);
int32_t attn_bwd_sm100_status(int* out);

// Reads and clears the device-side status word of the tcgen05 kernels (0 = no bounded wait gave up).
int32_t attn_fwd_sm100_status(int* out);

int32_t attn_fwd_dispatch(void* O, const void* Q, const void* K, const void* V, float* M, float* L,
                          const AttnParams& p, int32_t dtype, cudaStream_t st);
int64_t attn_bwd_workspace_bytes(int Dk, int Dv, int Sq, int Sk, int H, int Hkv, int B, int32_t dtype);
int32_t attn_bwd_dispatch(void* dQ, void* dK, void* dV, const void* Q, const void* K, const void* V,
                          const void* O, const void* dO, const float* M, const float* L, float* Delta,
                          void* workspace, const AttnParams& p, int32_t dtype, cudaStream_t st);

}  // namespace tylo
