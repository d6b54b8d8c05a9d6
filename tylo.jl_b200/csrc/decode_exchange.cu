// Sharded split-KV decode: merge of the per-GPU partials over peer memory, in one kernel.
//
// The reference's decode (src/attention/decode.jl:158-212) runs on one GPU: a split kernel writes
// per-split partials and mha_decode_combine merges them (algebra decode.jl:119-140).  When the KV
// cache of one sequence is sharded over GPUs, every GPU runs the split kernel on its own keys and
// the same algebra merges the per-GPU results.  Here that second level is ONE launch per GPU:
//
//   1. each CTA (one per (head, batch)) merges this GPU's split partials,
//   2. stores the merged record (Dv values, max, sum) into the receive buffer of every peer with
//      plain stores over NVLink, fences, and raises a per-(peer, head) flag with a release store,
//   3. waits — bounded — until the flags of all peers for this call have arrived in its own buffer,
//   4. merges the `world` records and writes the output.
//
// No collective library call and no host round trip sits between the split kernel and the result.
// Records are double-buffered by call parity, flags carry a call counter kept per head in the
// buffer itself, so the same launch can be replayed from a CUDA graph.
//
// The buffers come from cudaMalloc and are shared between the processes of one node through CUDA
// IPC handles (tylo_b200_peer_*): plain pointers at the C boundary, no torch types.
#include <cstring>

#include "decode_merge.cuh"

namespace tylo {

// One CTA of 1024 threads per (head, batch); see merge_partials for the thread layout.
template <typename T>
__global__ void __launch_bounds__(1024)
decode_exchange_kernel(T* __restrict__ O, const float* __restrict__ Op, const float* __restrict__ Mp,
                       const float* __restrict__ Lp, int n_splits, int64_t o_stride, int64_t ml_stride, int Dv,
                       int HB, const __grid_constant__ ExchangePeers peers, int rank, int world,
                       unsigned long long timeout_ns) {
  extern __shared__ __align__(16) float xsm[];
  float* res = xsm + 4096 + 64;
  const int hb = blockIdx.x;
  const int sl = threadIdx.y, tx = threadIdx.x, tid = sl * blockDim.x + tx;
  const ExchangeLayout lay = exchange_layout(world, HB, Dv);

  // ---- 1. this GPU's splits -> one record ----------------------------------------------------------
  dependency_wait();
  dependents_may_launch();
  float m, l;
  merge_partials<false>(Op + (size_t)hb * Dv, Mp + hb, Lp + hb, n_splits, o_stride, ml_stride, Dv, xsm, res, m, l);

  // ---- 2. push the record to every peer, then raise the flags ------------------------------------------
  uint32_t* self = reinterpret_cast<uint32_t*>(peers.buf[rank]);
  const uint32_t epoch = self[lay.epoch_off + hb] + 1u;     // call counter of this head; written back at the end
  const int par = (int)(epoch & 1u);
  for (int p = sl; p < world; p += blockDim.y) {
    float* rec = peers.buf[p] + lay.data_off + ((int64_t)(par * world + rank) * HB + hb) * lay.rec;
    if (tx * 4 < Dv) reinterpret_cast<float4*>(rec)[tx] = reinterpret_cast<const float4*>(res)[tx];
    if (tx == 0) *reinterpret_cast<float2*>(rec + Dv) = make_float2(m, l);
  }
  // The barrier orders the block's peer stores before the flag threads; their release store at system
  // scope is cumulative over everything ordered before it, so it publishes the whole record.
  __syncthreads();
  bool ok = true;
  if (tid < world) {
    st_release_sys(reinterpret_cast<uint32_t*>(peers.buf[tid]) + lay.flag_off + (int64_t)rank * HB + hb, epoch);
    // ---- 3. bounded wait for peer `tid`'s record of this call --------------------------------------------
    const uint32_t* f = self + lay.flag_off + (int64_t)tid * HB + hb;
    const unsigned long long t0 = global_ns();
    while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
      if (global_ns() - t0 > timeout_ns) { ok = false; break; }
      __nanosleep(64);
    }
  }
  ok = __syncthreads_and(ok);
  if (!ok) {
    // A peer never arrived: record it, keep the call counter in step, leave O untouched.
    if (tid == 0) { atomicMax(self, 1u + (uint32_t)hb); self[lay.epoch_off + hb] = epoch; }
    return;
  }

  // ---- 4. merge the records of all GPUs --------------------------------------------------------------------
  const float* mine = peers.buf[rank] + lay.data_off + ((int64_t)par * world * HB + hb) * lay.rec;
  const int64_t rstride = (int64_t)HB * lay.rec;
  float mg, lg;
  merge_partials<true>(mine, mine + Dv, mine + Dv + 1, world, rstride, rstride, Dv, xsm, res, mg, lg);
  if (tid < Dv) O[(size_t)hb * Dv + tid] = Elem<T>::from_f(res[tid]);
  if (tid == 0) self[lay.epoch_off + hb] = epoch;
}

template <typename T>
static int32_t decode_exchange_dispatch(void* O, const float* Op, const float* Mp, const float* Lp, int n_splits,
                                        int64_t o_stride, int64_t ml_stride, const ExchangePeers& peers, int rank,
                                        int world, int Dv, int H, int B, unsigned long long timeout_ns,
                                        cudaStream_t st) {
  const unsigned grid = (unsigned)((int64_t)H * B);
  const size_t smem = (size_t)merge_smem_floats(1024, Dv) * sizeof(float);
  TYLO_CUDA_OK(launch_overlapped(true, decode_exchange_kernel<T>, dim3(grid), merge_block(Dv), smem, st, (T*)O, Op, Mp, Lp,
                                 n_splits, o_stride, ml_stride, Dv, H * B, peers, rank, world, timeout_ns));
  return check_launch("decode_exchange");
}

}  // namespace tylo

using namespace tylo;

extern "C" int64_t tylo_b200_decode_exchange_bytes(int32_t world, int32_t Dv, int32_t H, int32_t B) {
  if (world <= 0 || world > kMaxExchangeWorld || Dv <= 0 || Dv > 512 || Dv % 4 != 0 || H <= 0 || B <= 0) return 0;
  return exchange_layout(world, H * B, Dv).total * 4;
}

extern "C" int32_t tylo_b200_decode_exchange(void* O, const float* O_partial, const float* M_partial,
                                             const float* L_partial, int32_t n_splits, int64_t o_stride,
                                             int64_t ml_stride, void* const* peer_buffers, int32_t rank,
                                             int32_t world, int32_t Dv, int32_t H, int32_t B, int32_t dtype,
                                             int64_t timeout_us, tylo_stream_t stream) {
  TYLO_REQUIRE(O && O_partial && M_partial && L_partial && peer_buffers, TYLO_ERR_INVALID_ARGUMENT,
               "decode_exchange: all pointers must be non-null");
  TYLO_REQUIRE(world >= 1 && world <= kMaxExchangeWorld, TYLO_ERR_UNSUPPORTED,
               "decode_exchange: world size %d outside 1..%d", world, kMaxExchangeWorld);
  TYLO_REQUIRE(rank >= 0 && rank < world, TYLO_ERR_INVALID_ARGUMENT, "decode_exchange: rank %d outside 0..%d", rank,
               world - 1);
  TYLO_REQUIRE(n_splits > 0 && Dv > 0 && H > 0 && B > 0, TYLO_ERR_INVALID_ARGUMENT,
               "decode_exchange: extents must be positive");
  TYLO_REQUIRE(Dv <= 512 && Dv % 4 == 0, TYLO_ERR_UNSUPPORTED,
               "decode_exchange: Dv (%d) must be a multiple of 4, at most 512", Dv);
  TYLO_REQUIRE(aligned16(O_partial) && o_stride % 4 == 0, TYLO_ERR_MISALIGNED,
               "decode_exchange: O_partial must be 16-byte aligned with o_stride a multiple of 4");
  TYLO_REQUIRE(o_stride >= (int64_t)H * B * Dv || n_splits == 1, TYLO_ERR_INVALID_ARGUMENT,
               "decode_exchange: o_stride smaller than one partial");
  TYLO_REQUIRE(ml_stride >= (int64_t)H * B || n_splits == 1, TYLO_ERR_INVALID_ARGUMENT,
               "decode_exchange: ml_stride smaller than one partial");
  ExchangePeers peers{};
  for (int r = 0; r < world; ++r) {
    TYLO_REQUIRE(peer_buffers[r] && aligned16(peer_buffers[r]), TYLO_ERR_INVALID_ARGUMENT,
                 "decode_exchange: peer buffer %d is null or not 16-byte aligned", r);
    peers.buf[r] = static_cast<float*>(peer_buffers[r]);
  }
  const unsigned long long timeout_ns =
      timeout_us > 0 ? (unsigned long long)timeout_us * 1000ull : 2000000000ull;   // default: two seconds
  TYLO_DISPATCH_DTYPE(dtype, T, return (decode_exchange_dispatch<T>(O, O_partial, M_partial, L_partial, n_splits,
                                                                    o_stride, ml_stride, peers, rank, world, Dv, H, B,
                                                                    timeout_ns, (cudaStream_t)stream)));
  return TYLO_OK;
}

extern "C" int32_t tylo_b200_decode_exchange_status(void* own_buffer, int32_t* code) {
  TYLO_REQUIRE(own_buffer && code, TYLO_ERR_INVALID_ARGUMENT, "decode_exchange_status: null argument");
  TYLO_CUDA_OK(cudaDeviceSynchronize());
  uint32_t v = 0, zero = 0;
  TYLO_CUDA_OK(cudaMemcpy(&v, own_buffer, 4, cudaMemcpyDeviceToHost));
  if (v != 0) TYLO_CUDA_OK(cudaMemcpy(own_buffer, &zero, 4, cudaMemcpyHostToDevice));
  *code = (int32_t)v;
  TYLO_REQUIRE(v == 0, TYLO_ERR_DEVICE_TIMEOUT,
               "decode_exchange: a peer's record did not arrive in time (first seen at head %d)", (int)v - 1);
  return TYLO_OK;
}

// ---- buffers shared between the processes of one node ------------------------------------------------------
extern "C" int32_t tylo_b200_peer_alloc(void** ptr, int64_t bytes) {
  TYLO_REQUIRE(ptr && bytes > 0, TYLO_ERR_INVALID_ARGUMENT, "peer_alloc: bad argument");
  TYLO_CUDA_OK(cudaMalloc(ptr, (size_t)bytes));
  TYLO_CUDA_OK(cudaMemset(*ptr, 0, (size_t)bytes));
  TYLO_CUDA_OK(cudaDeviceSynchronize());
  return TYLO_OK;
}
extern "C" int32_t tylo_b200_peer_free(void* ptr) {
  if (ptr) TYLO_CUDA_OK(cudaFree(ptr));
  return TYLO_OK;
}
extern "C" int32_t tylo_b200_peer_handle_bytes(void) { return (int32_t)sizeof(cudaIpcMemHandle_t); }
extern "C" int32_t tylo_b200_peer_export(const void* ptr, void* handle) {
  TYLO_REQUIRE(ptr && handle, TYLO_ERR_INVALID_ARGUMENT, "peer_export: null argument");
  cudaIpcMemHandle_t h;
  TYLO_CUDA_OK(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  std::memcpy(handle, &h, sizeof(h));
  return TYLO_OK;
}
extern "C" int32_t tylo_b200_peer_open(void** ptr, const void* handle) {
  TYLO_REQUIRE(ptr && handle, TYLO_ERR_INVALID_ARGUMENT, "peer_open: null argument");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  TYLO_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return TYLO_OK;
}
extern "C" int32_t tylo_b200_peer_close(void* ptr) {
  if (ptr) TYLO_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return TYLO_OK;
}
