// Merge of split-KV partials: the reference's mha_decode_combine algebra (src/attention/decode.jl:119-140)
// as a block-parallel reduction.  Used for the splits of one GPU and, once more, for the per-GPU records
// of a sharded sequence.
#pragma once

#include "common.cuh"

namespace tylo {

// Shared-memory floats merge_partials needs for a block of TX x SL threads and head dim Dv.
__host__ __device__ constexpr int merge_smem_floats(int threads, int Dv) { return threads * 4 + 2 * (threads / 32) + Dv + 64; }

// Block = (TX, SL) threads; thread (tx, sl) owns columns [4*tx, 4*tx+4) of partials sl, sl+SL, ...
// Each thread folds its partials online (running max, rescale), then the SL lanes are merged through
// shared memory.  All global loads of a thread are independent, so a block of 1024 threads keeps
// n_partials * Dv / 4 vector loads in flight at once instead of walking the partials serially.
//   o_base + s*o_stride : Dv normalised values of partial s (16-byte aligned, Dv % 4 == 0)
//   m_base + s*ml_stride, l_base + s*ml_stride : its max (log2 units) and sum
// Result: res[0..Dv) = merged, normalised values (shared memory); m_out, l_out on every thread.
// COHERENT: read with ld.global.cg (data another GPU has just written into this GPU's memory).
template <bool COHERENT>
__device__ __forceinline__ void merge_partials(const float* __restrict__ o_base, const float* __restrict__ m_base,
                                               const float* __restrict__ l_base, int n, int64_t o_stride,
                                               int64_t ml_stride, int Dv, float* sm, float* res, float& m_out,
                                               float& l_out) {
  const int TX = blockDim.x, SL = blockDim.y;
  const int tx = threadIdx.x, sl = threadIdx.y, tid = sl * TX + tx;
  const bool live = tx * 4 < Dv;
  float m = -INFINITY, l = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int s = sl; s < n; s += SL) {
    float ms, ls;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (COHERENT) {
      ms = __ldcg(m_base + s * ml_stride); ls = __ldcg(l_base + s * ml_stride);
      if (live) v = __ldcg(reinterpret_cast<const float4*>(o_base + s * o_stride) + tx);
    } else {
      ms = m_base[s * ml_stride]; ls = l_base[s * ml_stride];
      if (live) v = reinterpret_cast<const float4*>(o_base + s * o_stride)[tx];
    }
    const float mn = fmaxf(m, ms);
    const float a = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    const float w = (ms == -INFINITY) ? 0.f : ls * exp2f(ms - mn);
    acc.x = acc.x * a + w * v.x; acc.y = acc.y * a + w * v.y;
    acc.z = acc.z * a + w * v.z; acc.w = acc.w * a + w * v.w;
    l = l * a + w;
    m = mn;
  }
  float* sacc = sm;                       // [SL][TX*4]
  float* smx = sacc + SL * TX * 4;        // [SL]
  float* slx = smx + SL;                  // [SL]
  if (tx == 0) { smx[sl] = m; slx[sl] = l; }
  __syncthreads();
  float mg = -INFINITY;
  for (int k = 0; k < SL; ++k) mg = fmaxf(mg, smx[k]);
  float lg = 0.f;
  for (int k = 0; k < SL; ++k) lg += (smx[k] == -INFINITY) ? 0.f : slx[k] * exp2f(smx[k] - mg);
  const float f = (m == -INFINITY) ? 0.f : exp2f(m - mg);
  reinterpret_cast<float4*>(sacc)[tid] = make_float4(acc.x * f, acc.y * f, acc.z * f, acc.w * f);
  __syncthreads();
  if (tid < Dv) {
    float a = 0.f;
    for (int k = 0; k < SL; ++k) a += sacc[k * TX * 4 + tid];
    res[tid] = lg > 0.f ? a / lg : 0.f;
  }
  __syncthreads();
  m_out = mg; l_out = lg;
}

// ---- exchange of merged records between the GPUs of a node (sharded decode) ---------------------------
constexpr int kMaxExchangeWorld = 16;
struct ExchangePeers { float* buf[kMaxExchangeWorld]; };

struct ExchangeLayout {   // offsets in 4-byte words from the start of a rank's buffer
  int64_t epoch_off, flag_off, data_off, total;
  int rec;                // words per record: Dv values, max, sum, padded to a multiple of 4
};
__host__ __device__ inline ExchangeLayout exchange_layout(int world, int HB, int Dv) {
  ExchangeLayout l;
  l.rec = (Dv + 2 + 3) & ~3;
  l.epoch_off = 16;                                            // words 0..15: status word + reserved
  l.flag_off = l.epoch_off + ((HB + 15) & ~15);
  l.data_off = l.flag_off + (((int64_t)world * HB + 15) & ~15);
  l.total = l.data_off + (int64_t)2 * world * HB * l.rec;
  return l;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}


// Programmatic dependent launch: a merge kernel is launched while the split kernel before it on the
// stream is still running, so its launch latency and CTA placement overlap the split kernel's tail.
// dependency_wait() returns once the preceding kernel has finished and its writes are visible; it
// must precede the first read of that kernel's output.  dependents_may_launch() is the producer's
// side; it is a no-op when the next launch does not ask for overlap.
__device__ __forceinline__ void dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dependents_may_launch() { asm volatile("griddepcontrol.launch_dependents;"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Block shape for merge_partials: TX vector columns covering Dv (a power of two >= Dv/4, at least 32).
inline dim3 merge_block(int Dv) {
  const int tx = Dv <= 128 ? 32 : (Dv <= 256 ? 64 : 128);
  return dim3(tx, 1024 / tx);
}

}  // namespace tylo
