// placeholder replaced below
#include "attn_dispatch.cuh"
namespace tylo {
bool attn_fwd_sm100_supported(const AttnParams&, int32_t) { return false; }
int32_t attn_fwd_sm100(void*, const void*, const void*, const void*, float*, float*, const AttnParams&, int32_t,
                       cudaStream_t) {
  set_error("tcgen05 forward not built");
  return TYLO_ERR_UNSUPPORTED;
}
}  // namespace tylo
