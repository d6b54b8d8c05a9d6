/* libtylo_b200 — C ABI of the B200 (sm_100a) implementation of Tylo's transformer hot path.
 *
 * Each entry point replaces one launch group of the Tylo.jl package: the place where a
 * host wrapper such as `attention!` hands its arrays to `@cutile(blocks=…, kernel(…))`
 * (src/Tylo.jl:10-12).  The citation beside each declaration names the wrapper (and the
 * kernels it launches) that the entry point stands in for; paths are relative to the
 * Tylo.jl project root.
 *
 * Conventions
 *  - Arrays are dense, column-major (Julia) device buffers passed as raw pointers with
 *    explicit extents.  A Julia array of size (D, S, H, B) is the same memory as a
 *    C-contiguous array indexed [b][h][s][d].
 *  - Every buffer is owned by the caller.  Except where a declaration says otherwise the
 *    library allocates no device memory, never synchronises, and enqueues all work on
 *    the `stream` argument (a `cudaStream_t`; NULL = the legacy default stream).
 *  - Optional arrays are nullable pointers.
 *  - Every function returns a `tylo_status`; `tylo_b200_last_error()` gives the
 *    thread-local message of the last non-zero status.  Arguments are validated before
 *    anything is enqueued, so a non-zero status means no work was launched.
 *  - Data pointers must be 16-byte aligned (true of any CUDA allocation).
 */
#ifndef TYLO_B200_H
#define TYLO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TYLO_B200_VERSION 100 /* major*10000 + minor*100 + patch */

typedef enum {
  TYLO_OK = 0,
  TYLO_ERR_INVALID_ARGUMENT = 1, /* null / non-positive extent / inconsistent shapes (the wrappers' @assert) */
  TYLO_ERR_UNSUPPORTED = 2,      /* valid request this library has no kernel for (there is no fallback) */
  TYLO_ERR_MISALIGNED = 3,       /* a data pointer is not 16-byte aligned */
  TYLO_ERR_CUDA = 4,             /* a CUDA runtime/driver call failed; message holds its text */
  TYLO_ERR_NCCL = 5,             /* an NCCL call failed */
  TYLO_ERR_DEVICE_TIMEOUT = 6,   /* a bounded device-side wait gave up (see tylo_b200_device_status) */
  TYLO_ERR_WORKSPACE = 7         /* caller-provided workspace is too small */
} tylo_status;

typedef enum {
  TYLO_F32 = 0, TYLO_BF16 = 1, TYLO_F16 = 2,
  /* Float32 storage with the matrix products on the tensor cores, operands read as TF32 (sign, exponent,
   * 10 mantissa bits; fp32 accumulation and fp32 softmax) — the reference's default for Float32
   * (`tensorcore = TFloat32`, src/utils.jl:43-44).  Accepted by the attention and flex-attention FORWARD
   * entry points for head dims that are multiples of 4 up to 64; other head dims and OR-ed document terms are
   * computed in true fp32 there.  Every other entry point rejects it: pass TYLO_F32. */
  TYLO_F32_TF32 = 3
} tylo_dtype;

typedef void* tylo_stream_t; /* cudaStream_t */

int32_t tylo_b200_version(void);
const char* tylo_b200_status_string(int32_t status);
const char* tylo_b200_last_error(void);

/* Device-side health word of the tensor-core kernels.  Their internal waits (mbarriers between
 * the copy, MMA and softmax roles) are bounded; a wait that gives up stores a non-zero code and
 * the kernel drains instead of hanging.  This call synchronises the device, stores the code
 * (0 = healthy) in *code, clears it, and returns TYLO_ERR_DEVICE_TIMEOUT if it was non-zero.
 * No counterpart in the reference (its kernels never wait on one another). */
int32_t tylo_b200_device_status(int32_t* code);

/* ---- mod descriptors (src/attention/mods.jl) -------------------------------------------------
 * The Julia wrapper maps mod *types* to these plain structs by dispatch.  All enabled mask
 * terms are AND-ed (AndMask, mods.jl:151-157).  Positions are 0-based and absolute: query
 * position = row index + input_pos (flex.jl:41), key position = row index. */
#define TYLO_MASK_CAUSAL 1u    /* CausalMask: q >= kv (mods.jl:109-110) */
#define TYLO_MASK_SLIDING 2u   /* SlidingWindowMask(w): q >= kv && q <= kv + w (mods.jl:116-120) */
#define TYLO_MASK_DOCUMENT 4u  /* DocumentMask: doc_q[q] == doc_kv[kv] (mods.jl:141-147) */
#define TYLO_MASK_PREFIX 8u    /* PrefixMask(len): kv < len (mods.jl:127-131) */
#define TYLO_MASK_PREFIX_LM 16u /* prefix_lm(len) = causal | prefix (mods.jl:178) as one AND term */

typedef struct tylo_mask_desc {
  uint32_t flags;
  int32_t window;             /* SLIDING */
  int32_t prefix_len;         /* PREFIX / PREFIX_LM */
  int32_t reserved;
  const int32_t* doc_q;       /* DOCUMENT: device int32 ids indexed by absolute query position */
  const int32_t* doc_kv;      /* DOCUMENT: device int32 ids indexed by key position */
  int64_t doc_batch_stride;   /* 0: one table shared by every batch (the reference's semantics);
                                 otherwise element stride between per-batch tables */
  int64_t doc_q_len;          /* number of ids per table (bounds: input_pos + Sq <= doc_q_len) */
  int64_t doc_kv_len;
  const struct tylo_mask_desc* or_next; /* OrMask (mods.jl:164-167): NULL, or another conjunction OR-ed with this
                                           one — a mask tree is passed in disjunctive normal form, at most 4
                                           clauses.  Clauses of affine terms (causal, window, prefix) run on the
                                           tensor-core kernels as one key interval per clause and row; a clause
                                           with a DOCUMENT term sends the call to the fp32-arithmetic kernels.
                                           No block skipping with more than one clause.  prefix_lm keeps its own
                                           flag. */
} tylo_mask_desc;

#define TYLO_SCORE_ALIBI 1u         /* AliBiScore: s + slopes[h] * (q - kv), one slope per query head (mods.jl:205-209) */
#define TYLO_SCORE_SOFTCAP 2u       /* SoftCapScore: cap * tanh(s / cap) (mods.jl:194-198) */
#define TYLO_SCORE_SOFTCAP_FIRST 4u /* with soft cap and an additive mod: 0 = softcap ∘ additive (additive first),
                                       1 = additive ∘ softcap (mods.jl:244-249) */
#define TYLO_SCORE_BIAS 8u          /* BiasScore: s + bias[kv, q, mod1(h,nh), mod1(b,nb)] with LOCAL row indices
                                       q, kv (not shifted by input_pos) (mods.jl:212-237).  ALiBi and bias are both
                                       additive and sit at the same place of the chain. */

typedef struct {
  uint32_t flags;
  float cap;
  const float* slopes; /* device fp32, length H */
  float* d_slopes;     /* backward only, nullable: accumulates the slope gradient atomically
                          (grad_shadow semantics, mods.jl:296-303); caller zeroes it */
  const float* bias;   /* device fp32 (Sk, Sq, bias_heads, bias_batch), dense column-major; heads and batch
                          broadcast by mod1 when bias_heads < H or bias_batch < B */
  float* d_bias;       /* backward only, nullable: same shape, accumulated atomically (mods.jl:305-313);
                          caller zeroes it */
  int32_t bias_heads;
  int32_t bias_batch;
} tylo_score_desc;

/* ---- fused attention ---------------------------------------------------------------------------
 * attention! → mha_fwd (src/attention/attention.jl:219-262, kernel :6-88).
 * Q (Dk,Sq,H,B)  K (Dk,Sk,Hkv,B)  V (Dv,Sk,Hkv,B)  O (Dv,Sq,H,B);  scale = 1/sqrt(Dk).
 * M, L: optional fp32 (Sq,H,B) checkpoints: M = row max of s*scale*log2(e), L = sum exp2(.-M).
 * k_lengths / q_lengths: optional device int32 (B,) valid lengths (attention.jl:25-26,37-46,60).
 *   Keys at or beyond k_lengths[b] are masked; 64-row query blocks starting at or beyond
 *   q_lengths[b] are skipped (forward: their O/M/L rows stay untouched; backward: their gradient
 *   rows are zero).  As in the reference, masked elements meet probabilities of exactly zero inside
 *   matrix products, so K, V (and in the backward Q, O, dO) beyond the lengths must hold finite
 *   values, not uninitialised memory.
 * causal masks kv > q + input_pos.  dtype: storage type of Q,K,V,O.  fp32 storage is computed
 * in true fp32 (the reference's default rounds operands to TF32). */
int32_t tylo_b200_attention_fwd(void* O, const void* Q, const void* K, const void* V,
                                float* M, float* L,
                                const int32_t* k_lengths, const int32_t* q_lengths,
                                int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                int32_t H, int32_t Hkv, int32_t B,
                                int32_t input_pos, int32_t causal, int32_t dtype,
                                tylo_stream_t stream);

/* Bytes of caller-provided workspace the backward needs for these extents (0 is possible). */
int64_t tylo_b200_attention_bwd_workspace_bytes(int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                                int32_t H, int32_t Hkv, int32_t B, int32_t dtype);

/* ∇attention! → mha_bwd_preprocess + fill! + mha_bwd (attention.jl:297-357, kernels :90-198).
 * Overwrites dQ, dK, dV (no pre-zeroing needed).  Delta is the fp32 (Sq,H,B) scratch `Δ`;
 * dO_scaled is the reference's scratch `Ō′` (same shape/type as O): accepted for API
 * compatibility, may be NULL, not required to hold anything afterwards. */
int32_t tylo_b200_attention_bwd(void* dQ, void* dK, void* dV,
                                const void* Q, const void* K, const void* V,
                                const void* O, const void* dO,
                                const float* M, const float* L,
                                void* dO_scaled, float* Delta,
                                void* workspace, int64_t workspace_bytes,
                                const int32_t* k_lengths, const int32_t* q_lengths,
                                int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                int32_t H, int32_t Hkv, int32_t B,
                                int32_t input_pos, int32_t causal, int32_t dtype,
                                tylo_stream_t stream);

/* flex_attention! → flex_fwd (src/attention/flex.jl:312-383, kernel :22-105).
 * As attention_fwd plus score/mask mods; natural-base statistics: M = row max of the modded
 * score, L = sum exp(.-M); a fully masked query gives O = 0, M = -Inf, L = 0 (flex.jl:86-102).
 * qk_scale <= 0 selects the default 1/sqrt(Dk) (flex.jl:337).  mask/score may be NULL
 * (FullMask / NoOpScore).  block_sparse only permits skipping provably empty tiles. */
int32_t tylo_b200_flex_attention_fwd(void* O, const void* Q, const void* K, const void* V,
                                     float* M, float* L,
                                     const tylo_mask_desc* mask, const tylo_score_desc* score,
                                     int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                     int32_t H, int32_t Hkv, int32_t B,
                                     int32_t input_pos, float qk_scale, int32_t block_sparse,
                                     int32_t dtype, tylo_stream_t stream);

/* flex_attention!(...; block_mask) → flex_fwd_bm (src/attention/flex.jl:347-360, kernel :107-182):
 * the forward walks a host-built coarse BlockMask (src/attention/mods.jl:436-476) instead of the
 * analytic block range.  For query block i (tile_m rows) only the key blocks bm_idx[i][0 .. bm_count[i])
 * (tile_n keys each, 0-based ids) are visited; where bm_full[i][t] != 0 the mask mod is skipped and
 * only the key-length bound applies, elsewhere the mask mod is evaluated per pair; pairs in blocks
 * that are not listed contribute nothing.  bm_count (n_qb), bm_idx and bm_full (n_qb rows of
 * bm_stride entries — the reference's [n_kb, n_qb] column-major arrays) are device int32.
 * tile_m and tile_n must be multiples of 32; n_qb = ceil(Sq / tile_m); the block ids of one query
 * block must be distinct.  16-bit storage with a head dim that is a multiple of 8 up to 128 (and TYLO_F32_TF32
 * with a multiple of 4 up to 64) walks the
 * list on the tensor-core forward: key tiles from the smallest to the largest listed block, each 32-column chunk
 * of a warp's 32 rows looked up in the list (not listed: nothing kept; full: only the length bound; else the
 * mask mod); everything else runs on the fp32-arithmetic kernel. */
int32_t tylo_b200_flex_attention_fwd_block_mask(void* O, const void* Q, const void* K, const void* V,
                                                float* M, float* L,
                                                const tylo_mask_desc* mask, const tylo_score_desc* score,
                                                const int32_t* bm_count, const int32_t* bm_idx,
                                                const int32_t* bm_full, int32_t bm_stride,
                                                int32_t tile_m, int32_t tile_n,
                                                int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                                int32_t H, int32_t Hkv, int32_t B,
                                                int32_t input_pos, float qk_scale,
                                                int32_t dtype, tylo_stream_t stream);

/* Backward of the block-list forward above.  The reference has none (flex.jl:193-194: its list is per
 * query block and its backward loops over key blocks); here every (query tile, key tile) pair looks its
 * block up in the list, so the gradients are those of exactly the pairs the forward used: listed
 * blocks only, mask mod skipped where the block is marked full.  Arguments as flex_attention_bwd
 * (M, L from the block-list forward) plus the list. */
int32_t tylo_b200_flex_attention_bwd_block_mask(void* dQ, void* dK, void* dV,
                                                const void* Q, const void* K, const void* V,
                                                const void* O, const void* dO,
                                                const float* M, const float* L, float* Delta,
                                                void* workspace, int64_t workspace_bytes,
                                                const tylo_mask_desc* mask, const tylo_score_desc* score,
                                                const int32_t* bm_count, const int32_t* bm_idx,
                                                const int32_t* bm_full, int32_t bm_stride,
                                                int32_t tile_m, int32_t tile_n,
                                                int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                                int32_t H, int32_t Hkv, int32_t B,
                                                int32_t input_pos, float qk_scale,
                                                int32_t dtype, tylo_stream_t stream);

/* ∇flex_attention! → mha_bwd_preprocess + fill! + flex_bwd (flex.jl:445-511, kernel :197-289;
 * score VJPs mods.jl:288-319). */
int32_t tylo_b200_flex_attention_bwd(void* dQ, void* dK, void* dV,
                                     const void* Q, const void* K, const void* V,
                                     const void* O, const void* dO,
                                     const float* M, const float* L,
                                     void* dO_scaled, float* Delta,
                                     void* workspace, int64_t workspace_bytes,
                                     const tylo_mask_desc* mask, const tylo_score_desc* score,
                                     int32_t Dk, int32_t Dv, int32_t Sq, int32_t Sk,
                                     int32_t H, int32_t Hkv, int32_t B,
                                     int32_t input_pos, float qk_scale, int32_t block_sparse,
                                     int32_t dtype, tylo_stream_t stream);

/* ---- split-KV decode ---------------------------------------------------------------------------
 * decode_attention! → mha_decode_split_fwd + mha_decode_combine
 * (src/attention/decode.jl:158-212, kernels :28-143).
 * Q (Dk,H,B)  K (Dk,Sk,Hkv,B)  V (Dv,Sk,Hkv,B)  O (Dv,H,B)  lengths device int32 (B,).
 * Scratch (decode.jl:223-231): O_partial fp32 (Dv,H,B,n_splits) — normalised per split —,
 * M_partial (log2 units) and L_partial fp32 (H,B,n_splits).  Split s owns keys
 * [s*split_size, min((s+1)*split_size, len)), split_size = ceil(ceil(Sk/n_splits)/64)*64
 * (decode.jl:183, TILE_N = 64); an empty split writes (0, -Inf, 0). */
int32_t tylo_b200_decode_attention(void* O, const void* Q, const void* K, const void* V,
                                   const int32_t* lengths,
                                   float* O_partial, float* M_partial, float* L_partial,
                                   int32_t n_splits,
                                   int32_t Dk, int32_t Dv, int32_t Sk,
                                   int32_t H, int32_t Hkv, int32_t B,
                                   int32_t dtype, tylo_stream_t stream);

/* First half only (mha_decode_split_fwd, decode.jl:187-199): fills the partials. */
int32_t tylo_b200_decode_split(const void* Q, const void* K, const void* V,
                               const int32_t* lengths,
                               float* O_partial, float* M_partial, float* L_partial,
                               int32_t n_splits,
                               int32_t Dk, int32_t Dv, int32_t Sk,
                               int32_t H, int32_t Hkv, int32_t B,
                               int32_t dtype, tylo_stream_t stream);

/* Second half (mha_decode_combine, decode.jl:201-209, algebra :119-140).  `o_stride` and
 * `ml_stride` are the element strides between consecutive splits in O_partial and in
 * M_partial/L_partial (H*B*Dv and H*B for the scratch above); other strides let the same
 * routine merge per-GPU partials gathered into one buffer.  If O is non-NULL the merged
 * result is stored there in `dtype`.  If O_merged/M_merged/L_merged are non-NULL the merged
 * partial (normalised fp32 O, max, sum) is stored as well, for a further merge level. */
int32_t tylo_b200_decode_combine(void* O, float* O_merged, float* M_merged, float* L_merged,
                                 const float* O_partial, const float* M_partial,
                                 const float* L_partial,
                                 int32_t n_splits, int64_t o_stride, int64_t ml_stride,
                                 int32_t Dv, int32_t H, int32_t B,
                                 int32_t dtype, tylo_stream_t stream);

/* A split count that fills the GPU for these extents (the reference's default of 8 gives only
 * 8*Hkv*B blocks, decode.jl:163,187). */
int32_t tylo_b200_decode_suggest_splits(int32_t Sk, int32_t Hkv, int32_t B);

/* decode_attention in ONE launch (same arguments as tylo_b200_decode_attention plus `tickets`): the
 * split kernel's CTAs count themselves off per (kv head, batch); the last one of a group of eight
 * splits folds the group, the last group merges the groups (mha_decode_combine's algebra,
 * decode.jl:119-140) and writes O — no second kernel (decode.jl:187-209 launches two).
 * `tickets`: tylo_b200_decode_ticket_count(n_splits, Hkv, B) int32 words of device memory, zeroed
 * once by the caller; every call leaves them zero again.  Calls that share a ticket buffer (or the
 * partial buffers) must not overlap on the GPU.  Q, K, V must not be the output of a decode launch of
 * this library directly ahead on the same stream (the kernel starts reading them while such a launch
 * is still finishing).  With tickets == NULL, fp32 storage, head dims other than 64/128 or more than
 * 16 query heads per kv head the call is tylo_b200_decode_attention (two launches). */
int64_t tylo_b200_decode_ticket_count(int32_t n_splits, int32_t Hkv, int32_t B);
int32_t tylo_b200_decode_attention_fused(void* O, const void* Q, const void* K, const void* V,
                                         const int32_t* lengths,
                                         float* O_partial, float* M_partial, float* L_partial,
                                         int32_t* tickets, int32_t n_splits,
                                         int32_t Dk, int32_t Dv, int32_t Sk,
                                         int32_t H, int32_t Hkv, int32_t B,
                                         int32_t dtype, tylo_stream_t stream);

/* decode_attention over a PAGED KV cache (no counterpart in the reference, whose cache is one dense array
 * per sequence, decode.jl:158-165; the algorithm is the same split + merge).  K_pages / V_pages are pools of
 * pages of `page_size` keys, (Dk, page_size, Hkv, n_pages) and (Dv, page_size, Hkv, n_pages) column-major;
 * block_table is a device int32 (max_pages, B) column-major array: keys [i*page_size, (i+1)*page_size) of
 * sequence b live in page block_table[i, b].  Only entries below ceil(lengths[b] / page_size) are read.
 * One launch (tickets as for tylo_b200_decode_attention_fused); 16-bit storage, Dk == Dv in {64, 128}, at most
 * 16 query heads per kv head, page_size a multiple of 16 keys (32 at head dim 64).  Splits are taken over
 * page_size * max_pages keys. */
int32_t tylo_b200_decode_attention_paged(void* O, const void* Q, const void* K_pages, const void* V_pages,
                                         const int32_t* block_table, const int32_t* lengths,
                                         float* O_partial, float* M_partial, float* L_partial,
                                         int32_t* tickets, int32_t n_splits,
                                         int32_t page_size, int32_t max_pages,
                                         int32_t Dk, int32_t Dv, int32_t H, int32_t Hkv, int32_t B,
                                         int32_t dtype, tylo_stream_t stream);

/* decode_attention for callers that cannot supply scratch.  This entry has no counterpart in the
 * reference (there the scratch is always a caller-owned array, decode.jl:164,223-231).
 *
 * Who needs it: host code that may not allocate device memory at the point of the call — a
 * serving loop whose memory pool is frozen after start-up, a plugin inside a runtime that owns
 * all device memory, a callback without an allocator — and that has no spare buffer to pass.
 * Same arguments and result as tylo_b200_decode_attention, minus the three partial buffers: the
 * split partials are kept in a fixed fp32 array inside the library image
 * (tylo_b200_decode_static_scratch_floats() elements = 8 MiB, resident on every GPU that loads the
 * library, from load until the process exits).  The call allocates nothing and frees nothing.
 *
 *  - Limit: n_splits * B * H * (Dv + 2) must not exceed that element count; a larger request is
 *    refused with TYLO_ERR_WORKSPACE and a message (nothing is launched).
 *  - The first call on each device looks up the array's device address (a host-side symbol
 *    query, no allocation) with that device current; make that first call outside any stream
 *    capture.
 *  - All calls on a device share the one array and it keeps whatever the previous call left.
 *    The kernels overwrite every slot they later read, so no clearing is needed, but two calls
 *    whose GPU work overlaps (different streams, no ordering between them) race on it: order
 *    them on one stream or with events. */
int32_t tylo_b200_decode_attention_static(void* O, const void* Q, const void* K, const void* V,
                                          const int32_t* lengths, int32_t n_splits,
                                          int32_t Dk, int32_t Dv, int32_t Sk,
                                          int32_t H, int32_t Hkv, int32_t B,
                                          int32_t dtype, tylo_stream_t stream);
int64_t tylo_b200_decode_static_scratch_floats(void);

/* ---- decode with the KV cache of a sequence sharded over the GPUs of one node -------------------
 * No counterpart in the reference, which is single-GPU; the merge algebra is the reference's own
 * (mha_decode_combine, decode.jl:119-140) applied once more across GPUs.  Each GPU runs
 * tylo_b200_decode_split on its own key range, then tylo_b200_decode_exchange: ONE launch that
 * merges the local splits, stores the merged record into every peer's receive buffer over
 * NVLink (plain peer stores + a release flag per (peer, head)), waits — bounded — for the peers'
 * records of the same call and writes the final O (Dv,H,B) on every GPU.
 *
 * Receive buffers: one per GPU, tylo_b200_decode_exchange_bytes(world, Dv, H, B) bytes, zeroed,
 * mapped into every process (tylo_b200_peer_* below).  `peer_buffers` is a HOST array of `world`
 * device pointers, entry r = rank r's buffer as mapped in this process (entry `rank` = own).
 * All ranks must make the same sequence of calls on a buffer set (a per-head call counter lives
 * in the buffer); records are double-buffered, so calls may be replayed from a CUDA graph.
 * `timeout_us` bounds the wait for each peer (<= 0: two seconds).  When it runs out the kernel
 * leaves O untouched, sets the buffer's status word and returns; the context stays usable and
 * tylo_b200_decode_exchange_status reports TYLO_ERR_DEVICE_TIMEOUT once (reads and clears). */
int64_t tylo_b200_decode_exchange_bytes(int32_t world, int32_t Dv, int32_t H, int32_t B);
int32_t tylo_b200_decode_exchange(void* O, const float* O_partial, const float* M_partial,
                                  const float* L_partial,
                                  int32_t n_splits, int64_t o_stride, int64_t ml_stride,
                                  void* const* peer_buffers, int32_t rank, int32_t world,
                                  int32_t Dv, int32_t H, int32_t B, int32_t dtype,
                                  int64_t timeout_us, tylo_stream_t stream);
int32_t tylo_b200_decode_exchange_status(void* own_buffer, int32_t* code);

/* The sharded step in ONE launch per GPU: tylo_b200_decode_attention_fused on this GPU's key range
 * (`lengths_local` = live keys inside it, `Sk_local` = its allocated length) whose last CTA per
 * (kv head, batch) does what tylo_b200_decode_exchange does for the heads of that group: push the merged
 * record to every peer, raise the flags, wait (bounded by `timeout_us`, same status word) and merge the
 * `world` records into O.  Same receive buffers, same call counters: the two forms can be mixed call by
 * call as long as every rank makes the same sequence.  With tickets == NULL, and where the fused form does
 * not apply (see tylo_b200_decode_attention_fused), the call is split + exchange (two launches) — which is
 * also the faster form measured at 2 and 8 GPUs (the exchange kernel is placed under the split kernel's tail
 * and merges every head in a CTA of its own; 108 us against 123 us per step of a 1M-token cache at 8 GPUs). */
int32_t tylo_b200_decode_attention_sharded(void* O, const void* Q, const void* K, const void* V,
                                           const int32_t* lengths_local,
                                           float* O_partial, float* M_partial, float* L_partial,
                                           int32_t* tickets, int32_t n_splits,
                                           void* const* peer_buffers, int32_t rank, int32_t world,
                                           int32_t Dk, int32_t Dv, int32_t Sk_local,
                                           int32_t H, int32_t Hkv, int32_t B, int32_t dtype,
                                           int64_t timeout_us, tylo_stream_t stream);

/* Device buffers visible to every process of the node (CUDA IPC).  alloc: cudaMalloc + zero fill;
 * export: writes tylo_b200_peer_handle_bytes() opaque bytes to pass to the other processes by any
 * host channel; open: maps another process's buffer (peer access is enabled on first use);
 * close / free undo open / alloc.  Not called on the hot path. */
int32_t tylo_b200_peer_alloc(void** ptr, int64_t bytes);
int32_t tylo_b200_peer_free(void* ptr);
int32_t tylo_b200_peer_handle_bytes(void);
int32_t tylo_b200_peer_export(const void* ptr, void* handle);
int32_t tylo_b200_peer_open(void** ptr, const void* handle);
int32_t tylo_b200_peer_close(void* ptr);

/* ---- softmax -----------------------------------------------------------------------------------
 * softmax! → softmax_fwd / softmax_fwd_single (src/softmax/softmax.jl:96-105, kernels :6-33,:62-72).
 * X, Y (M,N): softmax along dim 1 (the contiguous one), one column per n. */
int32_t tylo_b200_softmax_fwd(void* Y, const void* X, int64_t M, int64_t N, int32_t dtype,
                              tylo_stream_t stream);
/* ∇softmax! → softmax_bwd / softmax_bwd_single (softmax.jl:127-136, kernels :35-60,:74-85):
 * dX = Y ∘ (dY − Σ Y∘dY). */
int32_t tylo_b200_softmax_bwd(void* dX, const void* dY, const void* Y, int64_t M, int64_t N,
                              int32_t dtype, tylo_stream_t stream);

/* ---- RMSNorm -----------------------------------------------------------------------------------
 * rms_norm! → rms_norm_fwd (src/norm/rms_norm.jl:115-128, kernel :6-32).
 * X, Y (M,N), W (M,), optional Rstd fp32 (N,):  y = x * rstd * (w + offset). */
int32_t tylo_b200_rms_norm_fwd(void* Y, const void* X, const void* W, float* Rstd,
                               int64_t M, int64_t N, float eps, float offset, int32_t dtype,
                               tylo_stream_t stream);
/* ∇rms_norm! → rms_norm_bwd_dx_partial_dw + rms_norm_bwd_dw (rms_norm.jl:162-185, kernels :34-99).
 * dW_partial is the fp32 (M, n_groups) scratch `W̄_partial`; it need not be zeroed and no lock
 * array is used (the reference serialises groups on a spin-lock, :68-78).  Overwrites dX, dW. */
int32_t tylo_b200_rms_norm_bwd(void* dX, void* dW, const void* dY, const void* X, const void* W,
                               const float* Rstd, float* dW_partial, int32_t n_groups,
                               int64_t M, int64_t N, float offset, int32_t dtype,
                               tylo_stream_t stream);

/* ---- LayerNorm ---------------------------------------------------------------------------------
 * layer_norm! → layer_norm_fwd (src/norm/layer_norm.jl:157-173, kernel :6-46).
 * Optional Mean, Rstd fp32 (N,). */
int32_t tylo_b200_layer_norm_fwd(void* Y, const void* X, const void* W, const void* Bias,
                                 float* Mean, float* Rstd,
                                 int64_t M, int64_t N, float eps, int32_t dtype,
                                 tylo_stream_t stream);
/* ∇layer_norm! → layer_norm_bwd_dx_partial_dwdb + layer_norm_bwd_dwdb
 * (layer_norm.jl:207-230, kernels :68-141).  dW_partial, dB_partial fp32 (M, n_groups). */
int32_t tylo_b200_layer_norm_bwd(void* dX, void* dW, void* dB, const void* dY, const void* X,
                                 const void* W, const float* Mean, const float* Rstd,
                                 float* dW_partial, float* dB_partial, int32_t n_groups,
                                 int64_t M, int64_t N, int32_t dtype, tylo_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TYLO_B200_H */
