// engine_gemma.cu -- tensor-parallel decode loop of a Gemma-4-E4B-shaped model (Q4_K
// weights, f16 KV cache, 5 sliding-window layers to 1 global layer, GeGLU FFN).
//
// Block order follows Hesper.Models.Gemma4.forwardBlock (Hesper/Models/Gemma4.lean:485):
// fused norm + q/k/v, RoPE + f16 KV write, decode attention, o_proj, post-attention norm
// then add, fused norm + gate/up GELU, down_proj, post-FFN norm then add; the reference's
// per-layer embeddings, MoE, vision/audio towers and per-head q/k norms are not part of
// the benchmark shape and are left out.
//
// Tensor parallelism (new: the reference is single-GPU): this rank holds a contiguous
// range of query heads with the KV head they attend to, the matching rows of gate/up and
// of the LM head, and the matching input columns of o_proj and down_proj.  The only
// exchange is one f32 sum all-reduce of hidden*batch elements after o_proj and after
// down_proj, and one u64 max all-reduce of batch argmax keys per token.
#include <algorithm>
#include <cstdlib>
#include <vector>

#include "common.cuh"

struct hb200_gemma {
  hb200_ctx* ctx;
  hb200_tp* tp;
  hb200_gemma_config cfg;
  std::vector<hb200_gemma_layer> layers;
  const void* embed;
  const void* lm_head;
  const float* final_norm;
  int B;
  int chunk_T;  // prompt positions per sequence one prefill pass takes (1: position by position)
  float *x, *x1, *q, *k, *v, *att, *o, *h, *logits;
  std::vector<__half*> kc, vc;  // per layer
  std::vector<int> slots;       // cache slots per layer (ring of window + chunk - 1, or max_seq)
  std::vector<int> win;         // attention window per layer (0: all positions)
  int32_t *pos, *len, *tok, *log_index, *token_log;
  unsigned long long* keys;
  double* rope_tab;  // [B * chunk_T][D/2][2] the pass's RoPE angles, shared by all layers
  void* attn_ws;
  size_t attn_ws_bytes;
  int log_stride;
};

namespace hb {

// keys[m] = max(keys[m], best (value, global index) of this rank's logits slice): ordered
// keys, so the maximum is the largest value and, among equals, the smallest index.  The grid
// is (chunks of `chunk` logits, tokens); every CTA folds its chunk and issues one atomicMax,
// whose result does not depend on the order of arrival.  keys[] must be zero on entry
// (keys_to_tokens_kernel leaves it so).
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t index) {
  if (!(v == v)) return 0ull;
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - index);
}
__global__ void __launch_bounds__(256) argmax_keys_kernel(const float* logits, int V, int voffset,
                                                          int chunk, unsigned long long* keys) {
  __shared__ unsigned long long red[8];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = logits + (size_t)m * V;
  const int i0 = blockIdx.x * chunk, i1 = min(V, i0 + chunk);
  unsigned long long best = 0;
  if ((reinterpret_cast<uintptr_t>(row + i0) & 15) == 0) {
    const int nvec = (i1 - i0) >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row + i0);
    for (int j = threadIdx.x; j < nvec; j += 256) {
      const float4 v = r4[j];
      const uint32_t g = (uint32_t)(i0 + 4 * j + voffset);
      unsigned long long k = argmax_key(v.x, g);
      best = k > best ? k : best;
      k = argmax_key(v.y, g + 1);
      best = k > best ? k : best;
      k = argmax_key(v.z, g + 2);
      best = k > best ? k : best;
      k = argmax_key(v.w, g + 3);
      best = k > best ? k : best;
    }
    for (int i = i0 + 4 * nvec + threadIdx.x; i < i1; i += 256) {
      const unsigned long long k = argmax_key(row[i], (uint32_t)(i + voffset));
      best = k > best ? k : best;
    }
  } else {
    for (int i = i0 + threadIdx.x; i < i1; i += 256) {
      const unsigned long long k = argmax_key(row[i], (uint32_t)(i + voffset));
      best = k > best ? k : best;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 1; i < 8; ++i) best = red[i] > best ? red[i] : best;
    if (best) atomicMax(keys + m, best);
  }
}

// Turns the reduced keys into tokens, logs them, and zeroes the keys for the next step.
__global__ void keys_to_tokens_kernel(unsigned long long* keys, int M, int32_t* tok,
                                      int32_t* log, const int32_t* log_index, int log_stride) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const unsigned long long k = keys[m];
  keys[m] = 0ull;
  const int32_t t = k ? (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull)) : 0;
  tok[m] = t;
  const int li = log_index[0];
  if (li >= 0 && li < log_stride) log[(size_t)m * log_stride + li] = t;
}

}  // namespace hb

using namespace hb;

namespace {

bool layer_is_global(const hb200_gemma_config& c, int l) {
  return c.global_every > 0 && (l + 1) % c.global_every == 0;
}

// One pass over all layers for T consecutive positions of every sequence (T = 1: a decode
// step; T > 1: a prompt chunk, d_tokens [nseq][T]).  Rows of every activation buffer are
// (sequence, token) pairs in that order.  Sliding-window layers keep a ring of window + chunk_T - 1
// slots, so the T positions written at the start of the pass overwrite nothing the pass's
// earliest query still attends to.  The LM head runs on each sequence's last row only.
int gemma_enqueue_step(hb200_gemma* m, const int32_t* d_tokens, bool lm_head, cudaStream_t st,
                       int T = 1) {
  const hb200_gemma_config& c = m->cfg;
  hb200_ctx* ctx = m->ctx;
  const int nseq = m->B, Hd = c.hidden, D = c.head_dim;
  const int B = nseq * T;  // rows
  const int qdim = c.local_q_heads * D, kvdim = c.local_kv_heads * D;
  const int32_t* toks = d_tokens ? d_tokens : m->tok;
  int rc = hb200_embed_lookup(ctx, m->embed, 0, c.vocab, Hd, toks, B, c.embed_scale, m->x, st);
  if (rc) return rc;
  rc = hb200_rope_table(ctx, m->pos, nseq, T, D, c.rope_base, m->rope_tab, st);
  if (rc) return rc;
  if (T > 1) {  // lengths after the chunk: pos + T (they stand at pos + 1 between passes)
    rc = hb200_add_i32(ctx, m->len, nseq, T - 1, st);
    if (rc) return rc;
  }
  // With one rank nothing has to be exchanged between a block's output projection and its
  // post-norm, so the post-norm + residual add runs inside the prologue of the NEXT matvec
  // launch (the o_proj / down_proj output stays in m->o until then): two launches fewer per
  // layer.  The last layer's post-FFN norm has no next matvec and runs on its own.
  const bool fold = m->tp == nullptr && getenv("HB200_NO_FOLD") == nullptr;
  for (int l = 0; l < c.n_layers; ++l) {
    const hb200_gemma_layer& L = m->layers[l];
    hb200_kquant_seg segs[3] = {
        {L.wq, nullptr, m->q, qdim}, {L.wk, nullptr, m->k, kvdim}, {L.wv, nullptr, m->v, kvdim}};
    if (fold && l > 0)  // x = x1 + rmsnorm(o) * post_ffn_norm of the previous layer
      rc = hb200_kquant_forward_multi_pre(ctx, HB200_FMT_Q4_K, segs, 3, Hd, m->o, B, m->x1,
                                          m->layers[l - 1].post_ffn_norm, m->x, L.attn_norm,
                                          c.rms_eps, st);
    else
      rc = hb200_kquant_forward_multi(ctx, HB200_FMT_Q4_K, segs, 3, Hd, m->x, B, L.attn_norm,
                                      c.rms_eps, st);
    if (rc) return rc;
    const bool ring = m->slots[l] < c.max_seq;
    rc = hb200_rope_kv_write_prefill_angles(ctx, m->q, m->k, m->v, m->kc[l], m->vc[l], m->pos,
                                            m->rope_tab, nseq, T, c.local_q_heads,
                                            c.local_kv_heads, D, m->slots[l], ring ? 1 : 0, st);
    if (rc) return rc;
    if (ring)  // position p sits in slot p % slots; the last `window` positions are alive
      rc = hb200_attn_ring(ctx, m->q, 0, m->kc[l], m->vc[l], m->len, nseq, T, c.local_q_heads,
                           c.local_kv_heads, D, m->slots[l], c.window, c.attn_scale, m->attn_ws,
                           m->attn_ws_bytes, m->att, st);
    else  // linear cache: a global layer, or a window too close to max_seq for a ring to pay
      rc = hb200_attn_prefill(ctx, m->q, 0, m->kc[l], m->vc[l], m->len, nseq, T, c.local_q_heads,
                              c.local_kv_heads, D, m->slots[l], m->win[l], c.attn_scale,
                              m->attn_ws, m->attn_ws_bytes, m->att, st);
    if (rc) return rc;
    rc = hb200_kquant_forward(ctx, HB200_FMT_Q4_K, L.wo, qdim, Hd, m->att, B, nullptr, 0.f, nullptr,
                              m->o, st);
    if (rc) return rc;
    if (fold) {  // x1 = x + rmsnorm(o) * post_attn_norm, then the gated FFN on x1
      rc = hb200_kquant_gateup_gelu_pre(ctx, HB200_FMT_Q4_K, L.wgate, L.wup, Hd, c.local_ffn, m->o,
                                        B, m->x, L.post_attn_norm, m->x1, L.ffn_norm, c.rms_eps,
                                        m->h, st);
    } else {
      rc = hb200_tp_allreduce_rmsnorm(m->tp, ctx, m->o, L.post_attn_norm, m->x, c.rms_eps, B, Hd,
                                      m->x1, st);
      if (rc) return rc;
      rc = hb200_kquant_gateup_gelu(ctx, HB200_FMT_Q4_K, L.wgate, L.wup, Hd, c.local_ffn, m->x1, B,
                                    L.ffn_norm, c.rms_eps, m->h, st);
    }
    if (rc) return rc;
    rc = hb200_kquant_forward(ctx, HB200_FMT_Q4_K, L.wdown, c.local_ffn, Hd, m->h, B, nullptr, 0.f,
                              nullptr, m->o, st);
    if (rc) return rc;
    if (!fold || l == c.n_layers - 1) {
      rc = hb200_tp_allreduce_rmsnorm(m->tp, ctx, m->o, L.post_ffn_norm, m->x1, c.rms_eps, B, Hd,
                                      m->x, st);
      if (rc) return rc;
    }
  }
  if (lm_head) {
    const float* xl = m->x;
    if (T > 1) {  // each sequence's last row, packed into x1 (free after the last layer)
      HB_CUDA(cudaMemcpy2DAsync(m->x1, sizeof(float) * Hd, m->x + (size_t)(T - 1) * Hd,
                                sizeof(float) * Hd * T, sizeof(float) * Hd, nseq,
                                cudaMemcpyDeviceToDevice, st));
      xl = m->x1;
    }
    rc = hb200_kquant_forward(ctx, HB200_FMT_Q4_K, m->lm_head, Hd, c.local_vocab, xl, nseq,
                              m->final_norm, c.rms_eps, nullptr, m->logits, st);
    if (rc) return rc;
    // enough CTAs to spread a single token's logits over the SMs, few atomics at large batch
    const int chunk = nseq <= 8 ? 2048 : 8192;
    HB_CUDA(launch_pdl(argmax_keys_kernel, dim3((c.local_vocab + chunk - 1) / chunk, nseq),
                       dim3(256), 0, st, ctx->pdl, (const float*)m->logits, c.local_vocab,
                       c.vocab_offset, chunk, m->keys));
    rc = hb200_tp_allreduce_max_u64(m->tp, m->keys, (size_t)nseq, st);
    if (rc) return rc;
    HB_CUDA(launch_pdl(keys_to_tokens_kernel, dim3((nseq + 63) / 64), dim3(64), 0, st, ctx->pdl,
                       m->keys, nseq, m->tok, m->token_log,
                       (const int32_t*)m->log_index, m->log_stride));
    rc = hb200_add_i32(ctx, m->log_index, 1, 1, st);
    if (rc) return rc;
  }
  // pos += T; len = pos + 1 again (the two arrays are adjacent: one launch for a decode step)
  if (T == 1) return hb200_add_i32(ctx, m->pos, 2 * nseq, 1, st);
  rc = hb200_add_i32(ctx, m->pos, nseq, T, st);
  if (rc) return rc;
  return hb200_add_i32(ctx, m->len, nseq, 1, st);
}

}  // namespace

extern "C" int hb200_gemma_create(hb200_ctx* ctx, hb200_tp* tp, const hb200_gemma_config* cfg,
                                  const hb200_gemma_layer* layers, const void* d_embed_bf16,
                                  const void* d_lm_head_q4k, const float* d_final_norm, int batch,
                                  int max_new_tokens, hb200_gemma** out) {
  HB_REQUIRE(ctx && cfg && layers && d_embed_bf16 && d_lm_head_q4k && d_final_norm && out,
             "gemma_create: null argument");
  HB_REQUIRE(batch >= 1 && batch <= 256, "gemma_create: batch %d outside 1..256", batch);
  HB_REQUIRE(cfg->hidden % 256 == 0 && cfg->local_ffn % 256 == 0 &&
                 (cfg->local_q_heads * cfg->head_dim) % 256 == 0 && cfg->local_kv_heads >= 1 &&
                 cfg->local_q_heads % cfg->local_kv_heads == 0,
             "gemma_create: local shapes must be multiples of the 256-weight super-block");
  *out = nullptr;
  hb200_gemma* m = new hb200_gemma();
  m->ctx = ctx;
  m->tp = tp;
  m->cfg = *cfg;
  m->layers.assign(layers, layers + cfg->n_layers);
  m->embed = d_embed_bf16;
  m->lm_head = d_lm_head_q4k;
  m->final_norm = d_final_norm;
  m->B = batch;
  m->log_stride = max_new_tokens > 0 ? max_new_tokens : 1;
  // prompt chunks: up to 256 rows per pass (the widest batched product), HB200_GEMMA_CHUNK caps
  // the positions per sequence (1 = position by position)
  int chunk_T = 256 / batch;
  if (const char* ev = getenv("HB200_GEMMA_CHUNK")) {
    const int cap = atoi(ev);
    if (cap >= 1 && cap < chunk_T) chunk_T = cap;
  }
  if (chunk_T < 1) chunk_T = 1;
  m->chunk_T = chunk_T;
  const int B = batch * chunk_T;  // rows of the activation buffers
  const int D = cfg->head_dim, qdim = cfg->local_q_heads * D, kvdim = cfg->local_kv_heads * D;
  cudaError_t e = cudaSuccess;
  auto A = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
  auto F = [&](float** p, size_t n) { A(cudaMalloc(reinterpret_cast<void**>(p), n * sizeof(float))); };
  F(&m->x, (size_t)B * cfg->hidden);
  F(&m->x1, (size_t)B * cfg->hidden);
  F(&m->o, (size_t)B * cfg->hidden);
  F(&m->q, (size_t)B * qdim);
  F(&m->k, (size_t)B * kvdim);
  F(&m->v, (size_t)B * kvdim);
  F(&m->att, (size_t)B * qdim);
  F(&m->h, (size_t)B * cfg->local_ffn);
  F(&m->logits, (size_t)batch * cfg->local_vocab);
  m->kc.assign(cfg->n_layers, nullptr);
  m->vc.assign(cfg->n_layers, nullptr);
  m->slots.assign(cfg->n_layers, 0);
  m->win.assign(cfg->n_layers, 0);
  int max_slots = 1;
  for (int l = 0; l < cfg->n_layers; ++l) {
    const bool glob = layer_is_global(*cfg, l) || cfg->window <= 0 || cfg->window >= cfg->max_seq;
    // a ring keeps the window plus the positions a prompt chunk adds before its first query
    // has looked back; if that is no shorter than the whole sequence the cache is linear
    m->slots[l] = glob ? cfg->max_seq : cfg->window + chunk_T - 1;
    if (m->slots[l] > cfg->max_seq) m->slots[l] = cfg->max_seq;
    m->win[l] = glob ? 0 : cfg->window;
    if (m->slots[l] > max_slots) max_slots = m->slots[l];
    const size_t n = (size_t)batch * cfg->local_kv_heads * m->slots[l] * D;
    A(cudaMalloc(reinterpret_cast<void**>(&m->kc[l]), n * sizeof(__half)));
    A(cudaMalloc(reinterpret_cast<void**>(&m->vc[l]), n * sizeof(__half)));
    if (e == cudaSuccess) e = cudaMemset(m->kc[l], 0, n * sizeof(__half));
    if (e == cudaSuccess) e = cudaMemset(m->vc[l], 0, n * sizeof(__half));
  }
  A(cudaMalloc(reinterpret_cast<void**>(&m->pos), sizeof(int32_t) * 2 * batch));
  m->len = m->pos ? m->pos + batch : nullptr;
  A(cudaMalloc(reinterpret_cast<void**>(&m->tok), sizeof(int32_t) * batch));
  A(cudaMalloc(reinterpret_cast<void**>(&m->log_index), sizeof(int32_t)));
  A(cudaMalloc(reinterpret_cast<void**>(&m->token_log), sizeof(int32_t) * (size_t)batch * m->log_stride));
  A(cudaMalloc(reinterpret_cast<void**>(&m->keys), sizeof(unsigned long long) * batch));
  A(cudaMemset(m->keys, 0, sizeof(unsigned long long) * batch));
  A(cudaMalloc(reinterpret_cast<void**>(&m->rope_tab), sizeof(double) * (size_t)B * D));
  m->attn_ws_bytes = hb200_attn_workspace_bytes(ctx, batch, cfg->local_q_heads,
                                                cfg->local_kv_heads, D, max_slots);
  // the split count, hence the partials, depend on the number of query tokens in a pass, and
  // not monotonically: size for every pass length a prompt can end with
  for (int T = 2; T <= chunk_T; ++T) {
    const size_t pw = hb200_attn_prefill_workspace_bytes(ctx, batch, T, cfg->local_q_heads,
                                                         cfg->local_kv_heads, D, max_slots);
    if (pw > m->attn_ws_bytes) m->attn_ws_bytes = pw;
  }
  A(cudaMalloc(&m->attn_ws, m->attn_ws_bytes));
  if (e != cudaSuccess) {
    hb200_gemma_destroy(m);
    return cuda_fail(e, "gemma_create allocation");
  }
  *out = m;
  return hb200_gemma_reset(m, nullptr);
}

extern "C" int hb200_gemma_destroy(hb200_gemma* m) {
  if (!m) return HB200_OK;
  cudaFree(m->x); cudaFree(m->x1); cudaFree(m->o); cudaFree(m->q); cudaFree(m->k); cudaFree(m->v);
  cudaFree(m->rope_tab);
  cudaFree(m->att); cudaFree(m->h); cudaFree(m->logits);
  for (auto p : m->kc) cudaFree(p);
  for (auto p : m->vc) cudaFree(p);
  cudaFree(m->pos); cudaFree(m->tok); cudaFree(m->log_index); cudaFree(m->token_log);
  cudaFree(m->keys); cudaFree(m->attn_ws);
  delete m;
  return HB200_OK;
}

extern "C" int hb200_gemma_reset(hb200_gemma* m, hb200_stream stream) {
  HB_REQUIRE(m != nullptr, "gemma_reset: null model");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B;
  std::vector<int32_t> init(2 * B, 0);
  for (int b = 0; b < B; ++b) init[B + b] = 1;
  HB_CUDA(cudaMemcpyAsync(m->pos, init.data(), sizeof(int32_t) * 2 * B, cudaMemcpyHostToDevice, st));
  HB_CUDA(cudaMemsetAsync(m->tok, 0, sizeof(int32_t) * B, st));
  HB_CUDA(cudaMemsetAsync(m->log_index, 0, sizeof(int32_t), st));
  HB_CUDA(cudaStreamSynchronize(st));
  return HB200_OK;
}

extern "C" int hb200_gemma_step(hb200_gemma* m, const int32_t* d_tokens, hb200_stream stream) {
  HB_REQUIRE(m != nullptr, "gemma_step: null model");
  return gemma_enqueue_step(m, d_tokens, true, static_cast<cudaStream_t>(stream));
}

extern "C" int hb200_gemma_prefill(hb200_gemma* m, const int32_t* d_tokens, int T, int want_token,
                                   hb200_stream stream) {
  HB_REQUIRE(m != nullptr && d_tokens != nullptr, "gemma_prefill: null argument");
  HB_REQUIRE(T >= 1 && T <= m->chunk_T, "gemma_prefill: %d positions per pass, at most %d", T,
             m->chunk_T);
  return gemma_enqueue_step(m, d_tokens, want_token != 0, static_cast<cudaStream_t>(stream), T);
}
extern "C" int hb200_gemma_chunk(const hb200_gemma* m) { return m ? m->chunk_T : 0; }

extern "C" const float* hb200_gemma_local_logits(const hb200_gemma* m) { return m ? m->logits : nullptr; }
extern "C" const int32_t* hb200_gemma_tokens(const hb200_gemma* m) { return m ? m->tok : nullptr; }

// Seeds every sequence's position (and length) without running the prompt: the KV cache keeps
// whatever it holds.  For throughput measurements at a given context length.
extern "C" int hb200_gemma_set_position(hb200_gemma* m, int pos, hb200_stream stream) {
  HB_REQUIRE(m != nullptr && pos >= 0 && pos < m->cfg.max_seq, "gemma_set_position: bad argument");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  std::vector<int32_t> init(2 * m->B, pos);
  for (int b = 0; b < m->B; ++b) init[m->B + b] = pos + 1;
  HB_CUDA(cudaMemcpyAsync(m->pos, init.data(), sizeof(int32_t) * 2 * m->B, cudaMemcpyHostToDevice, st));
  HB_CUDA(cudaStreamSynchronize(st));
  return HB200_OK;
}

extern "C" int hb200_gemma_generate(hb200_gemma* m, const int32_t* h_prompt, int prompt_len,
                                    int n_new, int use_graph, int32_t* h_out, float* ms_prefill,
                                    float* ms_decode, hb200_stream stream) {
  HB_REQUIRE(m && h_out, "gemma_generate: null argument");
  HB_REQUIRE(prompt_len >= 0 && n_new >= 1 && n_new <= m->log_stride,
             "gemma_generate: prompt_len=%d n_new=%d (log holds %d)", prompt_len, n_new, m->log_stride);
  HB_REQUIRE(prompt_len == 0 || h_prompt != nullptr, "gemma_generate: null prompt");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int B = m->B;
  cudaStream_t own = nullptr;
  if (st == nullptr) {  // the legacy default stream cannot be captured
    HB_CUDA(cudaStreamCreateWithFlags(&own, cudaStreamNonBlocking));
    st = own;
  }
  int rc = HB200_OK;
  int32_t* d_prompt = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaEvent_t e0, e1, e2;
  cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventCreate(&e2);
  auto cleanup = [&]() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    cudaEventDestroy(e0); cudaEventDestroy(e1); cudaEventDestroy(e2);
    if (d_prompt) cudaFree(d_prompt);
    if (own) cudaStreamDestroy(own);
  };
  cudaError_t e = cudaSuccess;
  // prompt_len == 0 continues from the current position (see hb200_gemma_set_position)
  if (prompt_len > 0) {
    rc = hb200_gemma_reset(m, st);
    if (rc) { cleanup(); return rc; }
    e = cudaMalloc(reinterpret_cast<void**>(&d_prompt), sizeof(int32_t) * (size_t)B * prompt_len);
    if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "prompt buffer"); }
    // chunk after chunk, each as [sequence][token of the chunk]
    std::vector<int32_t> pm((size_t)B * prompt_len);
    for (int p0 = 0; p0 < prompt_len; p0 += m->chunk_T) {
      const int T = std::min(m->chunk_T, prompt_len - p0);
      for (int b = 0; b < B; ++b)
        for (int t = 0; t < T; ++t)
          pm[(size_t)B * p0 + (size_t)b * T + t] = h_prompt[(size_t)b * prompt_len + p0 + t];
    }
    e = cudaMemcpyAsync(d_prompt, pm.data(), pm.size() * sizeof(int32_t), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "prompt upload"); }
    cudaStreamSynchronize(st);
  } else {
    HB_CUDA(cudaMemsetAsync(m->log_index, 0, sizeof(int32_t), st));
  }
  // the ranks reach this point after host work of different length; the exchanges that
  // follow wait with a deadline, so meet here first
  rc = hb200_tp_align(m->tp, st);
  if (rc) { cleanup(); return rc; }
  cudaEventRecord(e0, st);
  for (int p0 = 0; p0 < prompt_len; p0 += m->chunk_T) {
    const int T = std::min(m->chunk_T, prompt_len - p0);
    rc = gemma_enqueue_step(m, d_prompt + (size_t)B * p0, p0 + T == prompt_len, st, T);
    if (rc) { cleanup(); return rc; }
  }
  cudaEventRecord(e1, st);
  const int steps = prompt_len > 0 ? n_new - 1 : n_new;
  if (steps > 0) {
    if (use_graph) {
      e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
      if (e == cudaSuccess) {
        rc = gemma_enqueue_step(m, nullptr, true, st);
        cudaError_t e2c = cudaStreamEndCapture(st, &graph);
        if (rc) { cleanup(); return rc; }
        e = e2c;
      }
      if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
      if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "decode graph capture"); }
      rc = hb200_tp_align(m->tp, st);  // capture and instantiation take different time per rank
      if (rc) { cleanup(); return rc; }
      cudaEventRecord(e1, st);
      for (int s = 0; s < steps; ++s) {
        e = cudaGraphLaunch(exec, st);
        if (e != cudaSuccess) { cleanup(); return cuda_fail(e, "cudaGraphLaunch"); }
      }
    } else {
      for (int s = 0; s < steps; ++s) {
        rc = gemma_enqueue_step(m, nullptr, true, st);
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
  rc = hb200_ctx_check(m->ctx, st, &flags);
  cleanup();
  return rc;
}
