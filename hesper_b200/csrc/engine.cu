// engine.cu -- decode loop of a BitNet-b1.58-shaped model on one GPU, in C++ behind the C ABI.
//
// Mirrors Hesper.Models.BitNet.forwardSingleToken / generate (Hesper/Models/BitNet.lean:403,594)
// and the block order of TransformerBlock.forwardWithCache
// (Hesper/Layers/TransformerBlock.lean:439-485): per layer
//   [RMSNorm fused into] q/k/v BitLinear (one launch) -> RoPE + f16 KV write -> GQA decode
//   attention -> [sub-norm fused into] o BitLinear + residual -> [ffn norm fused into]
//   gate/up ReLU^2 GLU -> [sub-norm fused into] down BitLinear + residual,
// then the LM head over the tied bf16 embedding with the final norm fused in front and the
// greedy argmax fused behind.  Six launches per layer instead of the reference's ~18
// dispatches (ARCHITECTURE.md:107-131 of the reference).
//
// Everything a step needs from one token to the next lives on the device: the positions,
// the sequence lengths, the current tokens and the token log are device arrays advanced
// by kernels, so one captured CUDA graph is replayed for every decode step with no host
// writes in between (the reference rewrites a params buffer from the host every layer,
// Hesper/Layers/Attention.lean:1197-1206, and reads 4 bytes back per token, BitNet.lean:510-521).
#include <vector>

#include <cstdlib>

#include "common.cuh"

struct hb200_bitnet {
  hb200_ctx* ctx;
  hb200_bitnet_config cfg;
  std::vector<hb200_bitnet_layer> layers;
  const void* embed;
  int embed_dtype;
  const float* final_norm;
  int B;
  int Mmax;  // token rows the activation buffers hold: max(B, B * prefill chunk length)
  // device state
  float *x, *x1, *q, *k, *v, *att, *h, *logits, *xlast;
  double* rope_tab;  // [B][D/2][2] the step's RoPE angles, shared by all layers
  __half *kcache, *vcache;  // [layer][B][Hkv][max_seq][D]
  int32_t *pos, *len, *tok, *log_index, *token_log;
  void* lm_scratch;
  void* attn_ws;
  size_t attn_ws_bytes;
  int log_stride;
  bool want_logits;
};

using namespace hb;

namespace {

template <typename T>
cudaError_t dalloc(T** p, size_t n) {
  return cudaMalloc(reinterpret_cast<void**>(p), n * sizeof(T));
}

size_t layer_cache_elems(const hb200_bitnet* m) {
  return (size_t)m->B * m->cfg.n_kv_heads * m->cfg.max_seq * m->cfg.head_dim;
}

// One decode step for all B sequences, enqueued on `st`.
int enqueue_step(hb200_bitnet* m, const int32_t* d_tokens, bool lm_head, cudaStream_t st) {
  const hb200_bitnet_config& c = m->cfg;
  hb200_ctx* ctx = m->ctx;
  const int B = m->B, Hd = c.hidden, qdim = c.n_heads * c.head_dim, kvdim = c.n_kv_heads * c.head_dim;
  const int32_t* toks = d_tokens ? d_tokens : m->tok;
  int rc = hb200_embed_lookup(ctx, m->embed, m->embed_dtype, c.vocab, Hd, toks, B, 1.0f, m->x, st);
  if (rc) return rc;
  const float scale = 1.0f / sqrtf((float)c.head_dim);
  rc = hb200_rope_table(ctx, m->pos, B, 1, c.head_dim, c.rope_base, m->rope_tab, st);
  if (rc) return rc;
  for (int l = 0; l < c.n_layers; ++l) {
    const hb200_bitnet_layer& L = m->layers[l];
    hb200_bitlinear_seg segs[3] = {
        {L.wq, L.sq, nullptr, m->q, nullptr, qdim},
        {L.wk, L.sk, nullptr, m->k, nullptr, kvdim},
        {L.wv, L.sv, nullptr, m->v, nullptr, kvdim},
    };
    __half* kc = m->kcache + (size_t)l * layer_cache_elems(m);
    __half* vc = m->vcache + (size_t)l * layer_cache_elems(m);
    if (B == 1) {  // one launch: RoPE and the KV write are the matvec's epilogue
      rc = hb200_bitlinear_qkv_rope(ctx, segs, Hd, m->x, L.attn_norm, c.rms_eps, m->rope_tab,
                                    m->pos, kc, vc, c.n_heads, c.n_kv_heads, c.head_dim,
                                    c.max_seq, 0, st);
      if (rc) return rc;
    } else {
      rc = hb200_bitlinear_forward_multi(ctx, segs, 3, Hd, m->x, B, L.attn_norm, c.rms_eps, nullptr, st);
      if (rc) return rc;
      rc = hb200_rope_kv_write_angles(ctx, m->q, m->k, m->v, kc, vc, m->pos, m->rope_tab, B,
                                      c.n_heads, c.n_kv_heads, c.head_dim, c.max_seq, 0, st);
      if (rc) return rc;
    }
    rc = hb200_attn_decode(ctx, m->q, 0, kc, vc, m->len, B, c.n_heads, c.n_kv_heads, c.head_dim,
                           c.max_seq, 0, scale, m->attn_ws, m->attn_ws_bytes, m->att, st);
    if (rc) return rc;
    rc = hb200_bitlinear_forward(ctx, L.wo, L.so, qdim, Hd, m->att, B, L.attn_sub_norm, c.rms_eps,
                                 m->x, nullptr, nullptr, m->x1, st);
    if (rc) return rc;
    rc = hb200_bitlinear_gateup_relu2(ctx, L.wgate, L.sgate, L.wup, L.sup, Hd, c.ffn, m->x1, B,
                                      L.ffn_norm, c.rms_eps, m->h, st);
    if (rc) return rc;
    rc = hb200_bitlinear_forward(ctx, L.wdown, L.sdown, c.ffn, Hd, m->h, B, L.ffn_sub_norm,
                                 c.rms_eps, m->x1, nullptr, nullptr, m->x, st);
    if (rc) return rc;
  }
  if (lm_head) {
    rc = hb200_lmhead_argmax(ctx, m->embed, m->embed_dtype, c.vocab, Hd, m->x, B, m->final_norm,
                             c.rms_eps, m->want_logits ? m->logits : nullptr, m->tok,
                             m->lm_scratch, m->token_log, m->log_index, m->log_stride, st);
    if (rc) return rc;
    rc = hb200_add_i32(ctx, m->log_index, 1, 1, st);
    if (rc) return rc;
  }
  // pos and len are adjacent: one launch advances both
  return hb200_add_i32(ctx, m->pos, 2 * B, 1, st);
}

// Prompt chunk: T consecutive positions of every sequence in one pass (tokens [B][T] on the
// device, B*T <= 256).  The linear layers run batched on the tensor cores (bit-identical to
// the single-token kernels), RoPE/KV write and causal attention through their prefill entry
// points.  Positions advance by T.  With lm_head the last position's argmax is taken.
int enqueue_prefill_chunk(hb200_bitnet* m, const int32_t* d_tokens, int T, bool lm_head,
                          cudaStream_t st) {
  const hb200_bitnet_config& c = m->cfg;
  hb200_ctx* ctx = m->ctx;
  const int B = m->B, M = B * T, Hd = c.hidden;
  const int qdim = c.n_heads * c.head_dim, kvdim = c.n_kv_heads * c.head_dim;
  int rc = hb200_embed_lookup(ctx, m->embed, m->embed_dtype, c.vocab, Hd, d_tokens, M, 1.0f, m->x, st);
  if (rc) return rc;
  // len = pos + 1 between steps; the prefill entry points want the length after all T tokens
  rc = hb200_add_i32(ctx, m->len, B, T - 1, st);
  if (rc) return rc;
  const float scale = 1.0f / sqrtf((float)c.head_dim);
  for (int l = 0; l < c.n_layers; ++l) {
    const hb200_bitnet_layer& L = m->layers[l];
    hb200_bitlinear_seg segs[3] = {
        {L.wq, L.sq, nullptr, m->q, nullptr, qdim},
        {L.wk, L.sk, nullptr, m->k, nullptr, kvdim},
        {L.wv, L.sv, nullptr, m->v, nullptr, kvdim},
    };
    rc = hb200_bitlinear_forward_multi(ctx, segs, 3, Hd, m->x, M, L.attn_norm, c.rms_eps, nullptr, st);
    if (rc) return rc;
    __half* kc = m->kcache + (size_t)l * layer_cache_elems(m);
    __half* vc = m->vcache + (size_t)l * layer_cache_elems(m);
    rc = hb200_rope_kv_write_prefill(ctx, m->q, m->k, m->v, kc, vc, m->pos, B, T, c.n_heads,
                                     c.n_kv_heads, c.head_dim, c.max_seq, c.rope_base, st);
    if (rc) return rc;
    rc = hb200_attn_prefill(ctx, m->q, 0, kc, vc, m->len, B, T, c.n_heads, c.n_kv_heads, c.head_dim,
                            c.max_seq, 0, scale, m->attn_ws, m->attn_ws_bytes, m->att, st);
    if (rc) return rc;
    rc = hb200_bitlinear_forward(ctx, L.wo, L.so, qdim, Hd, m->att, M, L.attn_sub_norm, c.rms_eps,
                                 m->x, nullptr, nullptr, m->x1, st);
    if (rc) return rc;
    rc = hb200_bitlinear_gateup_relu2(ctx, L.wgate, L.sgate, L.wup, L.sup, Hd, c.ffn, m->x1, M,
                                      L.ffn_norm, c.rms_eps, m->h, st);
    if (rc) return rc;
    rc = hb200_bitlinear_forward(ctx, L.wdown, L.sdown, c.ffn, Hd, m->h, M, L.ffn_sub_norm,
                                 c.rms_eps, m->x1, nullptr, nullptr, m->x, st);
    if (rc) return rc;
  }
  if (lm_head) {
    // hidden state of each sequence's last position -> [B][Hd]
    HB_CUDA(cudaMemcpy2DAsync(m->xlast, (size_t)Hd * 4, m->x + (size_t)(T - 1) * Hd,
                              (size_t)T * Hd * 4, (size_t)Hd * 4, B, cudaMemcpyDeviceToDevice, st));
    rc = hb200_lmhead_argmax(ctx, m->embed, m->embed_dtype, c.vocab, Hd, m->xlast, B, m->final_norm,
                             c.rms_eps, m->want_logits ? m->logits : nullptr, m->tok,
                             m->lm_scratch, m->token_log, m->log_index, m->log_stride, st);
    if (rc) return rc;
    rc = hb200_add_i32(ctx, m->log_index, 1, 1, st);
    if (rc) return rc;
  }
  rc = hb200_add_i32(ctx, m->pos, B, T, st);  // pos += T
  if (rc) return rc;
  return hb200_add_i32(ctx, m->len, B, 1, st);  // len = pos + 1 again
}

}  // namespace

extern "C" int hb200_bitnet_create(hb200_ctx* ctx, const hb200_bitnet_config* cfg,
                                   const hb200_bitnet_layer* layers, const void* d_embed,
                                   int embed_dtype, const float* d_final_norm, int batch,
                                   int max_new_tokens, hb200_bitnet** out) {
  HB_REQUIRE(ctx && cfg && layers && d_embed && d_final_norm && out, "bitnet_create: null argument");
  HB_REQUIRE(batch >= 1 && batch <= 64, "bitnet_create: batch %d outside 1..64", batch);
  HB_REQUIRE(cfg->n_layers >= 1 && cfg->hidden % 128 == 0 && cfg->ffn % 128 == 0 &&
                 (cfg->n_heads * cfg->head_dim) % 128 == 0 && cfg->n_heads % cfg->n_kv_heads == 0,
             "bitnet_create: dimensions must be multiples of 128 and heads divisible");
  HB_REQUIRE(cfg->head_dim == 64 || cfg->head_dim == 128 || cfg->head_dim == 256,
             "bitnet_create: head_dim %d not in {64,128,256}", cfg->head_dim);
  *out = nullptr;
  hb200_bitnet* m = new hb200_bitnet();
  m->ctx = ctx;
  m->cfg = *cfg;
  m->layers.assign(layers, layers + cfg->n_layers);
  m->embed = d_embed;
  m->embed_dtype = embed_dtype;
  m->final_norm = d_final_norm;
  m->B = batch;
  m->log_stride = max_new_tokens > 0 ? max_new_tokens : 1;
  m->want_logits = false;
  const int B = batch, qdim = cfg->n_heads * cfg->head_dim, kvdim = cfg->n_kv_heads * cfg->head_dim;
  // prompt chunks of T = 256 / B positions run batched (the ternary products take them in
  // passes of 64 rows; RoPE, attention and the quantiser see all rows at once): the buffers
  // hold B * T token rows.  HB200_BITNET_CHUNK caps T.
  int Tmax = 256 / B;
  if (const char* ev = getenv("HB200_BITNET_CHUNK")) {
    const int cap = atoi(ev);
    if (cap >= 1 && cap < Tmax) Tmax = cap;
  }
  const size_t R = (size_t)B * (Tmax > 1 ? Tmax : 1);
  m->Mmax = (int)R;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
  A(dalloc(&m->x, R * cfg->hidden));
  A(dalloc(&m->x1, R * cfg->hidden));
  A(dalloc(&m->q, R * qdim));
  A(dalloc(&m->k, R * kvdim));
  A(dalloc(&m->v, R * kvdim));
  A(dalloc(&m->att, R * qdim));
  A(dalloc(&m->h, R * cfg->ffn));
  A(dalloc(&m->xlast, (size_t)B * cfg->hidden));
  A(dalloc(&m->rope_tab, (size_t)B * cfg->head_dim));  // [B][D/2] x (cos, sin)
  A(dalloc(&m->logits, (size_t)B * cfg->vocab));
  const size_t cache = (size_t)cfg->n_layers * layer_cache_elems(m);
  A(dalloc(&m->kcache, cache));
  A(dalloc(&m->vcache, cache));
  A(dalloc(&m->pos, (size_t)2 * B));  // pos[B] then len[B]
  m->len = m->pos ? m->pos + B : nullptr;
  A(dalloc(&m->tok, (size_t)B));
  A(dalloc(&m->log_index, 1));
  A(dalloc(&m->token_log, (size_t)B * m->log_stride));
  A(cudaMalloc(&m->lm_scratch, hb200_lmhead_scratch_bytes(B)));
  m->attn_ws_bytes = hb200_attn_workspace_bytes(ctx, B, cfg->n_heads, cfg->n_kv_heads,
                                                cfg->head_dim, cfg->max_seq);
  // the split count, hence the partials, depend on the query tokens of a pass, and not
  // monotonically: size for every chunk length a prompt can end with
  for (int T = 2; T <= Tmax; ++T) {
    const size_t pw = hb200_attn_prefill_workspace_bytes(ctx, B, T, cfg->n_heads,
                                                         cfg->n_kv_heads, cfg->head_dim, cfg->max_seq);
    if (pw > m->attn_ws_bytes) m->attn_ws_bytes = pw;
  }
  A(cudaMalloc(&m->attn_ws, m->attn_ws_bytes));
  if (e == cudaSuccess) e = cudaMemset(m->kcache, 0, cache * sizeof(__half));
  if (e == cudaSuccess) e = cudaMemset(m->vcache, 0, cache * sizeof(__half));
  if (e == cudaSuccess) e = cudaMemset(m->lm_scratch, 0, hb200_lmhead_scratch_bytes(B));
  if (e != cudaSuccess) {
    hb200_bitnet_destroy(m);
    return cuda_fail(e, "bitnet_create allocation");
  }
  *out = m;
  return hb200_bitnet_reset(m, nullptr);
}

extern "C" int hb200_bitnet_destroy(hb200_bitnet* m) {
  if (!m) return HB200_OK;
  cudaFree(m->x); cudaFree(m->x1); cudaFree(m->q); cudaFree(m->k); cudaFree(m->v);
  cudaFree(m->att); cudaFree(m->h); cudaFree(m->logits); cudaFree(m->kcache); cudaFree(m->vcache);
  cudaFree(m->xlast); cudaFree(m->rope_tab);
  cudaFree(m->pos); cudaFree(m->tok); cudaFree(m->log_index); cudaFree(m->token_log);
  cudaFree(m->lm_scratch); cudaFree(m->attn_ws);
  delete m;
  return HB200_OK;
}

extern "C" int hb200_bitnet_reset(hb200_bitnet* m, hb200_stream stream) {
  HB_REQUIRE(m != nullptr, "bitnet_reset: null model");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B;
  std::vector<int32_t> init(2 * B, 0);
  for (int b = 0; b < B; ++b) init[B + b] = 1;  // len = pos + 1
  HB_CUDA(cudaMemcpyAsync(m->pos, init.data(), sizeof(int32_t) * 2 * B, cudaMemcpyHostToDevice, st));
  HB_CUDA(cudaMemsetAsync(m->tok, 0, sizeof(int32_t) * B, st));
  HB_CUDA(cudaMemsetAsync(m->log_index, 0, sizeof(int32_t), st));
  HB_CUDA(cudaStreamSynchronize(st));
  return HB200_OK;
}

extern "C" int hb200_bitnet_step(hb200_bitnet* m, const int32_t* d_tokens, int want_logits,
                                 hb200_stream stream) {
  HB_REQUIRE(m != nullptr, "bitnet_step: null model");
  m->want_logits = want_logits != 0;
  return enqueue_step(m, d_tokens, true, static_cast<cudaStream_t>(stream));
}

extern "C" const float* hb200_bitnet_logits(const hb200_bitnet* m) { return m ? m->logits : nullptr; }
extern "C" const int32_t* hb200_bitnet_tokens(const hb200_bitnet* m) { return m ? m->tok : nullptr; }

extern "C" int hb200_bitnet_generate(hb200_bitnet* m, const int32_t* h_prompt, int prompt_len,
                                     int n_new, int use_graph, int32_t* h_out, float* ms_prefill,
                                     float* ms_decode, hb200_stream stream) {
  HB_REQUIRE(m && h_prompt && h_out, "bitnet_generate: null argument");
  HB_REQUIRE(prompt_len >= 1 && n_new >= 1 && n_new <= m->log_stride,
             "bitnet_generate: prompt_len=%d n_new=%d (log holds %d)", prompt_len, n_new,
             m->log_stride);
  HB_REQUIRE(prompt_len + n_new <= m->cfg.max_seq, "bitnet_generate: %d tokens exceed max_seq %d",
             prompt_len + n_new, m->cfg.max_seq);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B;
  int rc = hb200_bitnet_reset(m, stream);
  if (rc) return rc;
  // The legacy default stream cannot be captured: run the loop on a stream of our own then
  // (reset() above has synchronised with whatever the caller queued before).
  cudaStream_t own = nullptr;
  if (st == nullptr) {
    HB_CUDA(cudaStreamCreateWithFlags(&own, cudaStreamNonBlocking));
    st = own;
    stream = own;
  }
  m->want_logits = false;
  // prompt tokens in the order the prefill consumes them: chunks of T positions, each chunk
  // sequence-major [B][t]; with T = 1 that is position-major, a contiguous [B] slice per step
  const int T = m->Mmax / B > 1 ? m->Mmax / B : 1;
  int32_t* d_prompt = nullptr;
  HB_CUDA(cudaMalloc(&d_prompt, sizeof(int32_t) * (size_t)B * prompt_len));
  std::vector<int32_t> pm((size_t)B * prompt_len);
  for (int p0 = 0; p0 < prompt_len; p0 += T) {
    const int t = prompt_len - p0 < T ? prompt_len - p0 : T;
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < t; ++i)
        pm[(size_t)p0 * B + (size_t)b * t + i] = h_prompt[(size_t)b * prompt_len + p0 + i];
  }
  cudaError_t e = cudaMemcpyAsync(d_prompt, pm.data(), pm.size() * sizeof(int32_t),
                                  cudaMemcpyHostToDevice, st);
  cudaEvent_t e0, e1, e2;
  cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  auto cleanup = [&]() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    cudaFree(d_prompt);
    if (own) cudaStreamDestroy(own);
  };
  if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "prompt upload"); }
  // ---- prefill: the reference runs one single-token forward per prompt position
  //      (BitNet.generate :623-625); here chunks of T = 256 / B positions go through the
  //      batched kernels and causal prefill attention.  Only the last position needs the LM
  //      head, whose argmax is the first new token ----
  cudaEventRecord(e0, st);
  for (int p0 = 0; p0 < prompt_len; p0 += T) {
    const int t = prompt_len - p0 < T ? prompt_len - p0 : T;
    const bool last = p0 + t == prompt_len;
    rc = t > 1 ? enqueue_prefill_chunk(m, d_prompt + (size_t)p0 * B, t, last, st)
               : enqueue_step(m, d_prompt + (size_t)p0 * B, last, st);
    if (rc) { cleanup(); return rc; }
  }
  cudaEventRecord(e1, st);
  // ---- decode: n_new - 1 further steps feeding back the device-side argmax ----
  const int steps = n_new - 1;
  if (steps > 0) {
    if (use_graph) {
      e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
      if (e == cudaSuccess) {
        rc = enqueue_step(m, nullptr, true, st);
        cudaError_t e2c = cudaStreamEndCapture(st, &graph);
        if (rc) { cleanup(); return rc; }
        e = e2c;
      }
      if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
      if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "decode graph capture"); }
      cudaEventRecord(e1, st);  // capture and instantiation are not decode time
      for (int s = 0; s < steps; ++s) {
        e = cudaGraphLaunch(exec, st);
        if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "cudaGraphLaunch"); }
      }
    } else {
      for (int s = 0; s < steps; ++s) {
        rc = enqueue_step(m, nullptr, true, st);
        if (rc) { cleanup(); return rc; }
      }
    }
  }
  cudaEventRecord(e2, st);
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "decode"); }
  float a = 0.f, b2 = 0.f;
  cudaEventElapsedTime(&a, e0, e1);
  cudaEventElapsedTime(&b2, e1, e2);
  if (ms_prefill) *ms_prefill = a;
  if (ms_decode) *ms_decode = b2;
  std::vector<int32_t> log((size_t)B * m->log_stride);
  e = cudaMemcpy(log.data(), m->token_log, log.size() * sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "token log download"); }
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < n_new; ++i) h_out[(size_t)b * n_new + i] = log[(size_t)b * m->log_stride + i];
  uint32_t flags = 0;
  rc = hb200_ctx_check(m->ctx, stream, &flags);
  cleanup();
  return rc;
}
