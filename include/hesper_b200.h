/*
 * hesper_b200.h -- C ABI of the B200 (sm_100a) quantized-inference hot path.
 *
 * A drop-in for the three operator families that Hesper's Lean layers execute
 * through the PTX-emitting CUDA backend (native/cuda_bridge.cpp:374-444 behind
 * Hesper/Backend/CUDA.lean:523-660):
 *   - BitLinear ternary (i2_s) x int8 matvec       Hesper/Layers/BitLinear.lean
 *   - GGUF Q4_K / Q8_0 dequant-fused matvec         Hesper/Layers/Linear.lean
 *   - split-K GQA flash-attention decode (f16 KV)   Hesper/WGSL/FlashAttentionExperiments.lean
 *
 * Conventions (they follow the reference's external-kernel hook,
 * Hesper/Layers/Linear.lean:65-72 and Hesper/Backend/LlamaCppPTX.lean:138-155):
 *   - every pointer named d_* is a raw device address (a CUdeviceptr carried as
 *     a pointer); the caller owns every buffer, the library never frees,
 *     reallocates or retains them beyond the call;
 *   - `stream` is a CUstream / cudaStream_t (NULL = legacy default stream); all
 *     work is enqueued on it, nothing synchronises, allocates or calls back, so
 *     every launch can be captured into a CUDA graph;
 *   - weights are the verbatim GGUF payload bytes (i2_s packed bytes with a
 *     separate 4-byte f32 scale buffer; raw Q4_K / Q8_0 blocks);
 *   - each function returns HB200_OK or a negative code; hb200_last_error()
 *     gives the message (thread-local).  Nothing throws or aborts;
 *   - there is no CPU fallback: on a machine without an sm_100 GPU the calls
 *     fail with HB200_ERR_CUDA.
 */
#ifndef HESPER_B200_H
#define HESPER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define HB200_OK 0
#define HB200_ERR_INVALID (-1)     /* bad argument (shape, alignment, null) */
#define HB200_ERR_CUDA (-2)        /* a CUDA runtime call failed */
#define HB200_ERR_UNSUPPORTED (-3) /* shape or format outside what the kernels cover */
#define HB200_ERR_TIMEOUT (-4)     /* a bounded device-side wait gave up */

/* GGUF tensor type ids (Hesper/GGUF/Types.lean:86-132). */
#define HB200_FMT_Q8_0 8
#define HB200_FMT_Q4_K 12
#define HB200_FMT_I2_S 36

typedef struct hb200_ctx hb200_ctx;
typedef void *hb200_stream;

/* ---- context ------------------------------------------------------------- */

/* Replaces CUDAContext.init (Hesper/Backend/CUDA.lean:46; native/cuda_bridge.cpp:78-82)
 * for this path only: binds to `device` (its primary context), reads the SM
 * count, raises the kernels' dynamic shared-memory limits and allocates what the
 * operators need later: a 256-byte status block, 4096 arrival counters and 24 MB of
 * scratch (activation tiles, split-K partials of the batched paths).  No operator
 * allocates afterwards; a context serves one stream at a time (a call that arrives on
 * another stream than the previous scratch user's is ordered behind it with an event).
 * Environment: HB200_NO_PDL=1 launches without programmatic dependent launch,
 * HB200_NO_MMA=1 keeps the batched (>= 16 token) operators off the tensor-core kernels,
 * HB200_MV=0 / 2 keeps one-token matvecs off the mma.sync kernels / uses them wherever the
 * shape fits (default 1: ternary wherever two launches share an SM, k-quants where that holds
 * and it measured faster than the streaming kernel).
 * Measurement knobs of the decode loops and the exchange (same value on every rank):
 * HB200_NO_FOLD=1 keeps the post-norms of the Gemma-shape loop as launches of their own,
 * HB200_GEMMA_CHUNK=<n> / HB200_BITNET_CHUNK=<n> cap the prompt positions per sequence one
 * pass of the decode loops takes (default 256 / batch; 1 = position by position),
 * HB200_TP_TWO_SHOT_FROM=<tokens> moves the switch from the one-shot to the two-shot exchange,
 * HB200_TP_NO_LL=1 / HB200_TP_FUSE_MAX=<tokens> / HB200_TP_NO_PEER=1 select the
 * flag-after-data kernel, the unfused exchange above a batch size, or NCCL. */
int hb200_ctx_create(int device, hb200_ctx **out);

/* The same object inside the CUDA context that is current on the calling thread, for a host
 * that made its own context with the driver API -- Hesper does: cuCtxCreate on device 0,
 * native/cuda_bridge.cpp:78-82 -- and hands over CUdeviceptr / CUstream values that live in
 * it.  No cudaSetDevice, no primary-context retain: the device is the current context's,
 * every buffer of the library is allocated there, kernels are loaded there on first use.
 * The caller keeps that context current on the thread for every later call with this
 * handle and destroys the handle before the context.  Fails with HB200_ERR_INVALID when no
 * context is current. */
int hb200_ctx_create_current(hb200_ctx **out);
int hb200_ctx_destroy(hb200_ctx *ctx);

/* Message of the last failing call on this thread (never NULL).
 * Mirrors cudaErrorString in native/cuda_bridge.cpp:18-30. */
const char *hb200_last_error(void);

/* Library version: major*10000 + minor*100 + patch. */
int hb200_version(void);

/* Number of SMs the context sized its grids for. */
int hb200_ctx_sm_count(const hb200_ctx *ctx);

/* Synchronises `stream`, then reads and clears the device status block.
 * *flags != 0 means a kernel's bounded wait expired (HB200_ERR_TIMEOUT is
 * returned as well).  For tests and diagnostics; not on the hot path. */
int hb200_ctx_check(hb200_ctx *ctx, hb200_stream stream, uint32_t *flags);

/* Decode-attention arithmetic.
 *   FAST (default): the scaled query and the softmax weights are rounded to f16 for the
 *     tensor-core products (error ~5e-4, inside the 2e-3 bar).
 *   PRECISE: both are split into hi + lo f16 terms, twice the MMA work, error ~1e-6.
 *   EXACT: a slow one-warp-per-head kernel in which every f32 operation and its order are
 *     specified, so a CPU restatement reproduces it bit for bit.  For parity runs of a whole
 *     model only: its int8 re-quantisers amplify any 1e-6 difference into per-cent logit noise. */
#define HB200_ATTN_FAST 0
#define HB200_ATTN_PRECISE 1
#define HB200_ATTN_EXACT 2
int hb200_ctx_set_attn_mode(hb200_ctx *ctx, int mode);

/* Synchronises `stream` and copies the raw 64-word status block to `words`
 * without clearing it (word 0 = flags; the rest is kernel debug scratch). */
int hb200_ctx_read_status(hb200_ctx *ctx, hb200_stream stream, uint32_t words[64]);

/* ---- BitLinear: ternary i2_s weights x int8 activations ------------------- */

/* One output segment of a fused multi-matrix launch: several weight tensors
 * that consume the same activation vector (q/k/v; gate/up). */
typedef struct hb200_bitlinear_seg {
  const void *d_packed;    /* i2_s bytes, N*K/4, 16-byte aligned */
  const float *d_scale;    /* one f32: per-tensor scale */
  const float *d_residual; /* nullable, [M][N] added to the output */
  float *d_y;              /* [M][N] f32 output */
  int32_t *d_acc;          /* nullable, [M][N] raw int32 accumulators */
  int N;                   /* output rows of this tensor */
} hb200_bitlinear_seg;

/* y[m,n] = ((float)acc[m,n] * d[m]) * scale (+ residual[m,n]),
 * acc[m,n] = sum_k t[n,k] * q[m,k],  q = per-token absmax int8 of x
 * (d = amax/127, round-half-even), x optionally RMS-normalised first.
 *
 * Replaces BitLinear.forward (Hesper/Layers/BitLinear.lean:1226),
 * forwardWithResidual (:1308) and forwardFusedRMSNormResidual (:1370); the
 * arithmetic definition is Hesper/Layers/BitLinearSpec.lean:65-91 evaluated on
 * the int8 activations.
 *   d_x          [M][K] f32 activations
 *   d_rms_gamma  nullable [K]; when set x is replaced by RMSNorm(x)*gamma, eps = rms_eps
 *   d_act_scale  nullable [M]; receives d[m]
 * K must be a multiple of 128, 1 <= M <= 4096.  From 16 tokens on (and K <= 12288) the
 * product runs on the tensor cores in passes of up to 128 tokens (tcgen05 kind::i8, accumulators in tensor memory,
 * the M>1 role of Hesper/Layers/BitLinear.lean:122,869,994) with identical results. */
int hb200_bitlinear_forward(hb200_ctx *ctx, const void *d_packed, const float *d_scale,
                            int K, int N, const float *d_x, int M,
                            const float *d_rms_gamma, float rms_eps,
                            const float *d_residual, int32_t *d_acc,
                            float *d_act_scale, float *d_y, hb200_stream stream);

/* Same, for up to 4 tensors sharing x in ONE launch (fused q/k/v).  The
 * reference issues three BitLinear.forward calls (Hesper/Layers/Attention.lean:1191-1193). */
int hb200_bitlinear_forward_multi(hb200_ctx *ctx, const hb200_bitlinear_seg *segs,
                                  int nseg, int K, const float *d_x, int M,
                                  const float *d_rms_gamma, float rms_eps,
                                  float *d_act_scale, hb200_stream stream);

/* Fused q/k/v of ONE token with RoPE and the f16 KV-cache write in the kernel's epilogue: what
 * hb200_bitlinear_forward_multi (3 tensors, M = 1) followed by hb200_rope_kv_write_angles
 * (B = 1) compute, bit for bit, in one launch instead of two.  The reference issues three
 * BitLinear.forward calls, two RoPE launches and the KV writers
 * (Hesper/Layers/Attention.lean:1191-1224).
 *   segs[0..2]    q, k, v tensors; N = H*D, Hkv*D, Hkv*D.  segs[0].d_y receives the rotated q
 *                 (f32 [H][D]); segs[1].d_y / segs[2].d_y are f32 scratch rows that only the
 *                 two-launch route writes (taken for shapes the fused kernel does not cover)
 *   d_rope_table  [D/2][2] from hb200_rope_table (B = T = 1), d_pos [1] the token's position
 *   caches        [Hkv][cache_slots][D] f16 of the token's sequence; ring as in
 *                 hb200_rope_kv_write */
int hb200_bitlinear_qkv_rope(hb200_ctx *ctx, const hb200_bitlinear_seg *segs, int K,
                             const float *d_x, const float *d_rms_gamma, float rms_eps,
                             const double *d_rope_table, const int32_t *d_pos, void *d_k_cache,
                             void *d_v_cache, int H, int Hkv, int D, int cache_slots, int ring,
                             hb200_stream stream);

/* (cos, sin) in f64 of the RoPE angle of every (token, pair): d_table [B*T][D/2][2], token
 * t of sequence b at position d_pos[b] + t.  The angles are the same in every layer, so a
 * decode loop computes them once per step and hands them to hb200_rope_kv_write_angles,
 * which is hb200_rope_kv_write without the pow / sincos per element (same values). */
int hb200_rope_table(hb200_ctx *ctx, const int32_t *d_pos, int B, int T, int D, float rope_base,
                     double *d_table, hb200_stream stream);
int hb200_rope_kv_write_angles(hb200_ctx *ctx, float *d_q, const float *d_k, const float *d_v,
                               void *d_k_cache, void *d_v_cache, const int32_t *d_pos,
                               const double *d_table, int B, int H, int Hkv, int D,
                               int cache_slots, int ring, hb200_stream stream);

/* y[m,n] = relu(s_g*g[m,n])^2 * (s_u*u[m,n]) with g, u the two ternary matvecs.
 * Replaces BitLinear.forwardFusedGateUpReluSqrMul (Hesper/Layers/BitLinear.lean:1419,
 * kernel :553-621). */
int hb200_bitlinear_gateup_relu2(hb200_ctx *ctx, const void *d_packed_gate,
                                 const float *d_scale_gate, const void *d_packed_up,
                                 const float *d_scale_up, int K, int N, const float *d_x,
                                 int M, const float *d_rms_gamma, float rms_eps,
                                 float *d_y, hb200_stream stream);

/* ---- GGUF k-quants: Q4_K / Q8_0 dequant-fused matvec ----------------------- */

typedef struct hb200_kquant_seg {
  const void *d_blocks;    /* raw GGUF blocks, row-major [N][K/blk], 16-byte aligned */
  const float *d_residual; /* nullable [M][N] */
  float *d_y;              /* [M][N] */
  int N;
} hb200_kquant_seg;

/* y[m,n] = sum_k dequant(W)[n,k] * x[m,k] (+ residual).  f32 activations in and
 * f32 out; weights stay quantised in HBM.
 *
 * Replaces LinearLayer.forward / forwardDP4A (Hesper/Layers/Linear.lean:7115,5713)
 * and is what the hook Linear.llamaCppDp4aOverride (:65-72, consumed :5723-5740)
 * binds to: (inputF32Ptr, weightPtr, outputF32Ptr, inDim, outDim, quantTag).
 *   fmt  HB200_FMT_Q4_K or HB200_FMT_Q8_0; K a multiple of 256; 1 <= M <= 4096
 *   d_rms_gamma nullable: RMSNorm prologue as forwardFusedRMSNormLinear (:7897 region)
 * Up to 15 tokens stream the weights once per token through the dp4a kernel (activations
 * block-quantised to 16 bits, error ~2e-5).  From 16 tokens on the product runs on the
 * tensor cores, up to 256 tokens per pass: both formats are dequantised to f16 inside the
 * tcgen05 kernel; weights and activations rounded to f16 (every staged activation row
 * scaled by its own power of two), error ~4e-4 of max|y| (the bar of this path is 1e-3). */
int hb200_kquant_forward(hb200_ctx *ctx, int fmt, const void *d_blocks, int K, int N,
                         const float *d_x, int M, const float *d_rms_gamma, float rms_eps,
                         const float *d_residual, float *d_y, hb200_stream stream);

/* Up to 4 tensors sharing x in one launch: forwardFusedQKV / forwardFusedNormQKV /
 * forwardFusedKV (Hesper/Layers/Linear.lean:7413-7660). */
int hb200_kquant_forward_multi(hb200_ctx *ctx, int fmt, const hb200_kquant_seg *segs,
                               int nseg, int K, const float *d_x, int M,
                               const float *d_rms_gamma, float rms_eps,
                               hb200_stream stream);

/* y = gelu_tanh(x.Wg) * (x.Wu): forwardFusedGateUp / forwardFusedNormGateUp
 * (Hesper/Layers/Linear.lean:7295,7506); spec Hesper/Layers/FusedFFNSpec.lean:42-122. */
int hb200_kquant_gateup_gelu(hb200_ctx *ctx, int fmt, const void *d_blocks_gate,
                             const void *d_blocks_up, int K, int N, const float *d_x,
                             int M, const float *d_rms_gamma, float rms_eps, float *d_y,
                             hb200_stream stream);

/* The two calls above with a residual step in front, for layers that normalise a block's
 * output before adding it to the stream (post-attention / post-FFN norms, e.g.
 * Hesper/Models/Gemma4.lean:904-925 followed by the next block's fused norm + matvec):
 *   x' = d_pre_base + rmsnorm(d_o) * d_pre_gamma      (also written to d_x_out, [M][K])
 *   then hb200_kquant_forward_multi / hb200_kquant_gateup_gelu on x'.
 * The step has no launch of its own: up to 15 tokens it runs inside the matvec kernel's
 * prologue, from 16 tokens inside the kernel that stages the activations for the tensor-core
 * product (Q8_0 from 16 tokens: one hb200_rmsnorm launch).  d_x_out may alias neither input; all
 * arrays 16-byte aligned; rms_eps serves both norms. */
int hb200_kquant_forward_multi_pre(hb200_ctx *ctx, int fmt, const hb200_kquant_seg *segs,
                                   int nseg, int K, const float *d_o, int M,
                                   const float *d_pre_base, const float *d_pre_gamma,
                                   float *d_x_out, const float *d_rms_gamma, float rms_eps,
                                   hb200_stream stream);
int hb200_kquant_gateup_gelu_pre(hb200_ctx *ctx, int fmt, const void *d_blocks_gate,
                                 const void *d_blocks_up, int K, int N, const float *d_o,
                                 int M, const float *d_pre_base, const float *d_pre_gamma,
                                 float *d_x_out, const float *d_rms_gamma, float rms_eps,
                                 float *d_y, hb200_stream stream);

/* ---- decode attention ------------------------------------------------------ */

/* Bytes of scratch hb200_attn_decode needs for this shape (split-K partials). */
size_t hb200_attn_workspace_bytes(const hb200_ctx *ctx, int B, int H, int Hkv, int D,
                                  int max_seq);

/* GQA decode attention, one query token per sequence, f16 KV cache, split-K
 * over the sequence with all Q heads of a KV head sharing each K/V load.
 *
 * Replaces executeFlashAttentionV11 (Hesper/WGSL/FlashAttentionExperiments.lean:572)
 * = flashAttentionVecParamsKernelV11 (:45) + flashAttentionVecCombineKernel (:495).
 *   d_q        [B][H][D], f32 (q_is_f16 = 0, the reference's type) or f16
 *   d_k, d_v   [B][Hkv][max_seq][D] f16: per sequence the cache layout of
 *              Hesper/WGSL/FlashAttention.lean:590-597
 *   d_seqlens  [B] int32 valid positions per sequence (reference params[1] = cacheLen);
 *              the query is the last position, so all of them are visible
 *   window     0 = full attention; else only the last `window` positions
 *              (rule of flashAttentionSWAKernel, Hesper/WGSL/FlashAttention.lean:1621-1624)
 *   d_out      [B][H][D] f32
 * D in {64, 128, 256}, plus 32 on a slow one-warp-per-head kernel (the reference's smallest
 * golden case); H/Hkv in {1, 2, 4, 8}. */
int hb200_attn_decode(hb200_ctx *ctx, const void *d_q, int q_is_f16, const void *d_k,
                      const void *d_v, const int32_t *d_seqlens, int B, int H, int Hkv,
                      int D, int max_seq, int window, float scale, void *d_workspace,
                      size_t workspace_bytes, float *d_out, hb200_stream stream);


/* Causal prefill attention: T new query tokens per sequence against the same f16 cache,
 * which already holds them at positions seqlens[b]-T .. seqlens[b]-1 (written by
 * hb200_rope_kv_write_prefill).  Token t sees the positions before and including its own:
 * seqlens[b] - (T-1-t) of them (and of those only the last `window`, if set).
 * Replaces the prefill FlashAttention kernels (Hesper/WGSL/FlashAttention.lean:495-715).
 *   d_q, d_out  [B][T][H][D];  d_seqlens [B] lengths AFTER the T tokens were appended
 * From 8 tokens on (default attention mode) a CTA owns 64 query rows -- 64 / (H / Hkv) consecutive
 * tokens times the query heads of one KV head -- and walks the positions they see in tiles, so
 * a K/V tile is read once per 64 / (H / Hkv) tokens (role of flashAttentionBatchKernelF16,
 * Hesper/WGSL/FlashAttention.lean:601).  Shorter chunks and the PRECISE / EXACT modes run every
 * token as one decode query over its sequence's cache.  Linear caches (hb200_attn_ring for
 * rings).  T = 1 is hb200_attn_decode. */
size_t hb200_attn_prefill_workspace_bytes(const hb200_ctx *ctx, int B, int T, int H, int Hkv,
                                          int D, int max_seq);
int hb200_attn_prefill(hb200_ctx *ctx, const void *d_q, int q_is_f16, const void *d_k,
                       const void *d_v, const int32_t *d_seqlens, int B, int T, int H, int Hkv,
                       int D, int max_seq, int window, float scale, void *d_workspace,
                       size_t workspace_bytes, float *d_out, hb200_stream stream);

/* The same on a RING cache [B][Hkv][slots][D]: position p lives in slot p % slots (written by
 * hb200_rope_kv_write with ring != 0, or hb200_rope_kv_write_prefill_angles), d_seqlens are the
 * true lengths after the T tokens (they may exceed slots), and every query sees the last
 * `window` positions up to its own (rule of flashAttentionSWAKernel,
 * Hesper/WGSL/FlashAttention.lean:1621-1624).  Needs 1 <= window and window + T - 1 <= slots, so
 * that the T positions written before the call have not displaced anything the first of the T
 * queries still sees.  T = 1 is a decode step of a sliding-window layer.  Workspace:
 * hb200_attn_prefill_workspace_bytes(ctx, B, T, H, Hkv, D, slots). */
int hb200_attn_ring(hb200_ctx *ctx, const void *d_q, int q_is_f16, const void *d_k,
                    const void *d_v, const int32_t *d_seqlens, int B, int T, int H, int Hkv,
                    int D, int slots, int window, float scale, void *d_workspace,
                    size_t workspace_bytes, float *d_out, hb200_stream stream);

/* Decode attention for callers that cannot hand over scratch memory.  No counterpart in
 * the reference (there the Lean side allocates the V11 partial buffers with the model).
 *
 * Same operator, arguments and results as hb200_attn_decode, minus the workspace: the
 * split-K partials go to a fixed HB200_ATTN_STATIC_SCRATCH_BYTES array that is part of
 * the library image, so the call never allocates or frees device memory, neither directly
 * nor through a library.  It is meant for hosts where a device allocation at this point is
 * not an option: a runtime that has already handed the whole GPU to its own buffer pool
 * (Hesper's pooled CUDABuffer allocator works that way), or a thread that may not stall on
 * the device-wide synchronisation cudaMalloc can imply.  It still makes ordinary CUDA
 * runtime calls (device query, kernel launch), so it is not for host callbacks.
 *
 *   - Shapes whose partials exceed the array are refused with HB200_ERR_UNSUPPORTED and
 *     a message naming both sizes; use hb200_attn_decode for those.  With the current split
 *     rule (about two waves of resident CTAs, at most 64 splits) no supported shape reaches
 *     the limit -- the decode sweeps up to batch 64 x 32768 positions at 8/2 heads, D = 256
 *     stay below 5 MiB -- so the check guards future split rules.
 *   - The first call of a context looks up the array's device address (with the context's
 *     device current).  Make that first call before any stream capture is started on the
 *     thread.
 *   - All calls on a device share the one array and find the previous call's partials in
 *     it; that is harmless (every value read is written first within the same call), but
 *     two calls that overlap on the GPU, e.g. on different streams, race on it.  Keep calls
 *     to this entry point ordered on one stream per device.
 *   - Every GPU that loads the library holds the array for the lifetime of the process. */
#define HB200_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
int hb200_attn_decode_static(hb200_ctx *ctx, const void *d_q, int q_is_f16, const void *d_k,
                             const void *d_v, const int32_t *d_seqlens, int B, int H, int Hkv,
                             int D, int max_seq, int window, float scale, float *d_out,
                             hb200_stream stream);

/* ---- decode-step glue ------------------------------------------------------- */

/* y[m] = table[ids[m]] * scale as f32.  dtype: 0 = bf16, 1 = f16, 2 = f32.
 * Replaces embeddingLookupKernel (Hesper/Layers/Embedding.lean:116). */
int hb200_embed_lookup(hb200_ctx *ctx, const void *d_table, int dtype, long V, int K,
                       const int32_t *d_ids, int M, float scale, float *d_y,
                       hb200_stream stream);

/* y[m] = (d_add ? d_add[m] : 0) + RMSNorm(x[m]) * gamma.  Replaces RMSNorm.forward and
 * forwardNormThenAdd (Hesper/Layers/RMSNorm.lean:219,794); formula
 * Hesper/Training/VerifiedBackward.lean:95-99. */
int hb200_rmsnorm(hb200_ctx *ctx, const float *d_x, const float *d_gamma, const float *d_add,
                  float eps, int M, int K, float *d_y, hb200_stream stream);

/* NeoX RoPE (pairs d, d + D/2; angle pos * base^(-2i/D)) on q in place and on k, then
 * k and v packed to f16 and written into the caches at the token's position.
 * Replaces ropeKernelDynamic (Hesper/Layers/RoPE.lean:189) + the f16 KV writers
 * fusedRopeKAndCacheWriteKernelF16 / kvWriteBatchKernelF16 (Hesper/Layers/Attention.lean:701-945).
 *   d_q [B][H][D] f32, d_k / d_v [B][Hkv][D] f32, caches [B][Hkv][cache_slots][D] f16,
 *   d_pos [B] int32.  ring != 0 writes slot pos % cache_slots (sliding-window layers). */
int hb200_rope_kv_write(hb200_ctx *ctx, float *d_q, const float *d_k, const float *d_v,
                        void *d_k_cache, void *d_v_cache, const int32_t *d_pos, int B, int H,
                        int Hkv, int D, int cache_slots, int ring, float rope_base,
                        hb200_stream stream);

/* The prompt-chunk writer below with the angles taken from hb200_rope_table (d_table
 * [B*T][D/2][2]) and, with ring != 0, slot = position % cache_slots (T <= cache_slots). */
int hb200_rope_kv_write_prefill_angles(hb200_ctx *ctx, float *d_q, const float *d_k,
                                       const float *d_v, void *d_k_cache, void *d_v_cache,
                                       const int32_t *d_pos0, const double *d_table, int B, int T,
                                       int H, int Hkv, int D, int cache_slots, int ring,
                                       hb200_stream stream);

/* The same for T new tokens per sequence (prompt chunk): d_q [B][T][H][D], d_k / d_v
 * [B][T][Hkv][D], token t of sequence b is at position d_pos0[b] + t.  Linear caches only.
 * Replaces the batched RoPE + kvWriteBatchKernelF16 of the prefill path
 * (Hesper/Layers/Attention.lean:809-945). */
int hb200_rope_kv_write_prefill(hb200_ctx *ctx, float *d_q, const float *d_k, const float *d_v,
                                void *d_k_cache, void *d_v_cache, const int32_t *d_pos0, int B,
                                int T, int H, int Hkv, int D, int cache_slots, float rope_base,
                                hb200_stream stream);

/* Greedy argmax over [M][V] logits, first strict maximum.  Replaces argmaxKernel
 * (Hesper/Models/BitNet.lean:456-479). */
int hb200_argmax(hb200_ctx *ctx, const float *d_logits, long V, int M, int32_t *d_out,
                 hb200_stream stream);

/* LM head over a 16-bit table [V][K] (dtype 0 = bf16, 1 = f16) with the final RMSNorm
 * fused in front (d_rms_gamma nullable) and the greedy argmax fused behind.
 * Replaces executeMatMulTransposeF16Shared + gpuArgmax (Hesper/Models/BitNet.lean:437-521).
 * 1 <= M <= 64; from 16 tokens on (K a multiple of 64) the table is streamed once through
 * the tensor cores (tcgen05 kind::f16, activations split into two 16-bit terms so that
 * f32-activation accuracy is kept).
 *   d_logits   nullable [M][V]
 *   d_argmax   [M] token ids
 *   d_scratch  hb200_lmhead_scratch_bytes(M) bytes, zero before the first call (the
 *              call leaves it zero again)
 *   d_token_log / d_log_index / log_stride  nullable: token m is also stored at
 *              d_token_log[m*log_stride + *d_log_index] */
size_t hb200_lmhead_scratch_bytes(int M);
int hb200_lmhead_argmax(hb200_ctx *ctx, const void *d_table, int dtype, long V, int K,
                        const float *d_x, int M, const float *d_rms_gamma, float rms_eps,
                        float *d_logits, int32_t *d_argmax, void *d_scratch,
                        int32_t *d_token_log, const int32_t *d_log_index, int log_stride,
                        hb200_stream stream);

/* y = relu(g)^2 * u (reluSqrMulKernel, Hesper/WGSL/Elementwise.lean:320) and
 * y = gelu_tanh(g) * u (geluMulKernel, Hesper/Models/Gemma4/Kernels.lean:26). */
int hb200_relu2_mul(hb200_ctx *ctx, const float *d_gate, const float *d_up, long n, float *d_y,
                    hb200_stream stream);
int hb200_gelu_mul(hb200_ctx *ctx, const float *d_gate, const float *d_up, long n, float *d_y,
                   hb200_stream stream);

/* a[i] += delta for n int32 counters kept on the device (positions, lengths), so a
 * captured decode step advances without host writes.  The reference rewrites its
 * params buffer from the host every layer (Hesper/Layers/Attention.lean:1197-1206). */
int hb200_add_i32(hb200_ctx *ctx, int32_t *d_a, int n, int delta, hb200_stream stream);

/* ---- BitNet-b1.58-shaped decode loop --------------------------------------- */

/* Shape of the model (Hesper/Models/BitNet.lean:189-199 for the 2B configuration). */
typedef struct hb200_bitnet_config {
  int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, max_seq;
  float rope_base, rms_eps;
} hb200_bitnet_config;

/* Device pointers of one transformer block; all borrowed.  Weights are i2_s bytes, each
 * with its one-f32 scale buffer; norms are f32 vectors. */
typedef struct hb200_bitnet_layer {
  const float *attn_norm, *attn_sub_norm, *ffn_norm, *ffn_sub_norm;
  const void *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
  const float *sq, *sk, *sv, *so, *sgate, *sup, *sdown;
} hb200_bitnet_layer;

typedef struct hb200_bitnet hb200_bitnet;

/* Allocates the activations, the f16 KV cache [layer][batch][kv_head][max_seq][head_dim]
 * and the device-side counters for `batch` sequences decoded in lock step; nothing is
 * allocated afterwards.  d_embed is the [vocab][hidden] table (dtype 0 = bf16, 1 = f16),
 * also used as the tied LM head.  max_new_tokens sizes the device token log.
 * Replaces BitNet model construction + createCachedLayerBuffers / KV cache creation
 * (Hesper/Models/BitNet.lean:358-398). */
int hb200_bitnet_create(hb200_ctx *ctx, const hb200_bitnet_config *cfg,
                        const hb200_bitnet_layer *layers, const void *d_embed, int embed_dtype,
                        const float *d_final_norm, int batch, int max_new_tokens,
                        hb200_bitnet **out);
int hb200_bitnet_destroy(hb200_bitnet *m);

/* Positions back to 0 (the cache content is simply overwritten as decoding proceeds). */
int hb200_bitnet_reset(hb200_bitnet *m, hb200_stream stream);

/* Enqueues ONE decode step for all sequences: forwardSingleToken
 * (Hesper/Models/BitNet.lean:403) + gpuArgmax (:456).  d_tokens [batch] int32 are the
 * input tokens, or NULL to feed back the previous step's argmax.  The step advances the
 * device-side positions itself and is capturable.  want_logits != 0 also stores the
 * [batch][vocab] logits (hb200_bitnet_logits). */
int hb200_bitnet_step(hb200_bitnet *m, const int32_t *d_tokens, int want_logits,
                      hb200_stream stream);
const float *hb200_bitnet_logits(const hb200_bitnet *m);
const int32_t *hb200_bitnet_tokens(const hb200_bitnet *m);

/* generate (Hesper/Models/BitNet.lean:594): prefill as single-token forwards over
 * h_prompt [batch][prompt_len] (host), then n_new greedy tokens per sequence into h_out
 * [batch][n_new] (host).  With use_graph the decode step is captured once and replayed.
 * ms_prefill / ms_decode (nullable) receive device times; ms_decode covers the n_new - 1
 * steps after the prefill (the first new token is the prefill's argmax). */
int hb200_bitnet_generate(hb200_bitnet *m, const int32_t *h_prompt, int prompt_len, int n_new,
                          int use_graph, int32_t *h_out, float *ms_prefill, float *ms_decode,
                          hb200_stream stream);

/* ---- tensor parallelism (no counterpart in the reference: it is single-GPU) ------------- */

typedef struct hb200_tp hb200_tp;

/* One process per GPU.  Rank 0 makes the 128-byte id (ncclGetUniqueId), the host program
 * carries it to the other ranks by any means, then every rank calls hb200_tp_init.  NCCL is
 * loaded at run time (dlopen), so a single-GPU process needs no NCCL at all. */
int hb200_tp_unique_id(unsigned char out[128]);
int hb200_tp_init(hb200_ctx *ctx, int rank, int nranks, const unsigned char id[128],
                  hb200_tp **out);
int hb200_tp_destroy(hb200_tp *tp);
int hb200_tp_rank(const hb200_tp *tp);
int hb200_tp_size(const hb200_tp *tp);

/* In-place sum of n f32 over the ranks (the exchange after a row-split o_proj / down_proj)
 * and in-place max of n u64 (argmax keys after a column-split LM head), enqueued on `stream`
 * (capturable).  A NULL tp or a 1-rank communicator is a no-op. */
int hb200_tp_allreduce_f32(hb200_tp *tp, float *d_buf, size_t n, hb200_stream stream);
int hb200_tp_allreduce_max_u64(hb200_tp *tp, unsigned long long *d_buf, size_t n,
                               hb200_stream stream);

/* One-shot all-reduce over peer memory for the small exchanges of decode (optional; without
 * it every exchange goes through NCCL).  Each rank exports the handle of its exchange
 * buffer (hb200_tp_peer_handle_bytes() bytes, a CUDA IPC handle), the host program gathers
 * the handles of all ranks in rank order, every rank attaches.  From then on
 * hb200_tp_allreduce_* of up to 2560 x 64 floats run as ONE kernel per rank: push the
 * vector into every rank's buffer over NVLink, wait for the peers' flags (bounded; expiry
 * shows as HB200_ERR_TIMEOUT in hb200_ctx_check), add in rank order -- so all ranks hold
 * bit-identical sums.  Plain peer loads and stores only.  At most 8 ranks of one node, one
 * process per GPU.  All ranks must attach, or none. */
size_t hb200_tp_peer_handle_bytes(void);
int hb200_tp_peer_export(hb200_tp *tp, unsigned char *out_handle);
int hb200_tp_peer_attach(hb200_tp *tp, const unsigned char *all_handles);
int hb200_tp_peer_attached(const hb200_tp *tp);

/* The exchange and the RMSNorm that follows it in the decode loop as one operator:
 * y = d_add + RMSNorm(sum over ranks of d_x) * gamma.  With the peer buffers attached it is
 * ONE kernel, a CTA per token.  Up to 32 tokens every rank pushes its row to all peers, waits,
 * adds in rank order and normalises (one shot).  From 33 tokens (and K <= 3072, M <= 256) the
 * exchange is two-shot by token: a row goes only to the rank that owns the token, which
 * reduces, normalises and sends the finished row to everybody -- 2(W-1)/W of the payload per
 * rank instead of W-1 times it.  Otherwise it is hb200_tp_allreduce_f32 + hb200_rmsnorm (d_x
 * then holds the sum).  tp NULL or one rank: hb200_rmsnorm alone.  The path depends only on
 * M, K, the rank count and the switches read at hb200_tp_init (HB200_TP_FUSE_MAX,
 * HB200_TP_TWO_SHOT_FROM, HB200_TP_NO_LL: same values on every rank); arrays that are not
 * 16-byte aligned are an error, not a reason to take another path than the peers. */
int hb200_tp_allreduce_rmsnorm(hb200_tp *tp, hb200_ctx *ctx, float *d_x, const float *d_gamma,
                               const float *d_add, float eps, int M, int K, float *d_y,
                               hb200_stream stream);

/* Host-side health check of the communicator (ncclCommGetAsyncError): a peer that died or
 * never joined shows up here or as an error of the next collective, not as a GPU fault. */
int hb200_tp_check(hb200_tp *tp);

/* Bound of every device-side wait of the exchange kernels (default 1000 ms).  A wait that
 * runs out raises the context's status flag (hb200_ctx_check then returns
 * HB200_ERR_TIMEOUT), the kernel returns, and later exchanges of that context look once and
 * go on, so a run with a missing peer ends quickly and the GPU stays usable. */
int hb200_tp_set_timeout_ms(hb200_tp *tp, int ms);

/* Host-side meeting point of the ranks (one 4-byte NCCL all-reduce, then a stream
 * synchronisation).  Call it after rank-local host work of unknown length -- allocation,
 * upload, graph capture -- and before a run of exchanges, whose waits are bounded: the
 * decode loops do. */
int hb200_tp_align(hb200_tp *tp, hb200_stream stream);

/* ---- Gemma-4-E4B-shaped tensor-parallel decode loop ----------------------------------
 * (benchmark shape: 42 layers, hidden 2560, 8/2 heads of 256, GeGLU FFN 10240, vocab 262144) */

/* Global shape plus this rank's share.  Layer l is a global-attention layer when
 * (l+1) % global_every == 0, else a sliding-window layer whose cache is a ring of `window`
 * slots.  Shape source: Hesper/Models/Gemma4/Config.lean:19-45, simplified to one head size
 * and plain layers (no per-layer embeddings, MoE, towers or per-head q/k norms). */
typedef struct hb200_gemma_config {
  int n_layers, hidden, head_dim, vocab, max_seq, window, global_every;
  int local_q_heads, local_kv_heads, local_ffn, local_vocab, vocab_offset;
  float rope_base, rms_eps, attn_scale, embed_scale;
} hb200_gemma_config;

/* This rank's shards, all Q4_K, device pointers, borrowed.  wq/wk/wv/wgate/wup/lm_head are
 * row ranges of the full tensors (contiguous bytes); wo and wdown are column ranges, i.e.
 * for every output row the super-blocks of this rank's input slice, stored contiguously. */
typedef struct hb200_gemma_layer {
  const float *attn_norm, *post_attn_norm, *ffn_norm, *post_ffn_norm;
  const void *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;
} hb200_gemma_layer;

typedef struct hb200_gemma hb200_gemma;

/* Replaces Gemma4 model construction (Hesper/Models/Gemma4.lean:78-123) for the benchmark
 * shape.  tp may be NULL on one GPU.  d_embed_bf16 is the full [vocab][hidden] table. */
int hb200_gemma_create(hb200_ctx *ctx, hb200_tp *tp, const hb200_gemma_config *cfg,
                       const hb200_gemma_layer *layers, const void *d_embed_bf16,
                       const void *d_lm_head_q4k, const float *d_final_norm, int batch,
                       int max_new_tokens, hb200_gemma **out);
int hb200_gemma_destroy(hb200_gemma *m);
int hb200_gemma_reset(hb200_gemma *m, hb200_stream stream);
/* Positions of all sequences := pos without running a prompt (cache content stays as is);
 * for throughput measurements at a given context length. */
int hb200_gemma_set_position(hb200_gemma *m, int pos, hb200_stream stream);
/* One decode step on every rank: Gemma4.forwardSingleToken (Hesper/Models/Gemma4.lean:2558). */
int hb200_gemma_step(hb200_gemma *m, const int32_t *d_tokens, hb200_stream stream);
/* One pass over T consecutive prompt positions of every sequence: Gemma4.forwardPrefillBatch
 * (Hesper/Models/Gemma4.lean:1333).  d_tokens [batch][T], 1 <= T <= hb200_gemma_chunk(m)
 * (= 256 / batch rows per pass, capped by HB200_GEMMA_CHUNK when the model is created).  Same
 * kernels as a step at batch * T rows: batched products, RoPE + KV write of the T positions,
 * causal attention (sliding-window layers keep a ring of window + chunk - 1 slots).
 * want_token != 0 also runs the LM head on each sequence's last position and logs its token. */
int hb200_gemma_prefill(hb200_gemma *m, const int32_t *d_tokens, int T, int want_token,
                        hb200_stream stream);
int hb200_gemma_chunk(const hb200_gemma *m);
const float *hb200_gemma_local_logits(const hb200_gemma *m);
const int32_t *hb200_gemma_tokens(const hb200_gemma *m);
/* Gemma4.generate (Hesper/Models/Gemma4.lean:3212).  prompt_len = 0 continues from the
 * current position and decodes n_new tokens. */
int hb200_gemma_generate(hb200_gemma *m, const int32_t *h_prompt, int prompt_len, int n_new,
                         int use_graph, int32_t *h_out, float *ms_prefill, float *ms_decode,
                         hb200_stream stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* HESPER_B200_H */
