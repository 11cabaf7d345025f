// glue.cu -- the small kernels that sit between the three headline operators inside a
// decode step: embedding gather, RMSNorm (+add), NeoX RoPE fused with the f16 KV-cache
// write, the bf16/f16 LM-head matvec with fused greedy argmax, and the GLU epilogues.
// Reference counterparts: embeddingLookupKernel (Hesper/Layers/Embedding.lean:116),
// rmsNormFusedKernel (Hesper/Layers/RMSNorm.lean:219), ropeKernelDynamic
// (Hesper/Layers/RoPE.lean:189) + fusedRopeKAndCacheWriteKernelF16 / kvWriteBatchKernelF16
// (Hesper/Layers/Attention.lean:701-945), matMulTransposeF16SharedKernel
// (Hesper/WGSL/MatMul.lean:356), argmaxKernel (Hesper/Models/BitNet.lean:456),
// reluSqrMulKernel (Hesper/WGSL/Elementwise.lean:320), geluMulKernel
// (Hesper/Models/Gemma4/Kernels.lean:26).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common.cuh"
#include "rope.cuh"

namespace hb {

// ---- embedding gather ---------------------------------------------------------------

// dtype: 0 = bf16, 1 = f16, 2 = f32
__global__ void embed_kernel(const void* table, int dtype, const int32_t* ids, int K, long V,
                             float scale, float* y) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x;
  long id = ids[m];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  float* out = y + (size_t)m * K;
  if (dtype == 2) {
    const float* row = static_cast<const float*>(table) + (size_t)id * K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) out[k] = row[k] * scale;
  } else {
    const uint16_t* row = static_cast<const uint16_t*>(table) + (size_t)id * K;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
      const uint16_t b = row[k];
      const float v = dtype == 0 ? __uint_as_float((uint32_t)b << 16)
                                 : __half2float(__ushort_as_half(b));
      out[k] = v * scale;
    }
  }
}

// ---- RMSNorm (+ add) -------------------------------------------------------------------

// y[m] = (add ? add[m] : 0) + x[m] / sqrt(mean(x[m]^2) + eps) * gamma.  One CTA per row.
__global__ void rmsnorm_kernel(const float* x, const float* gamma, const float* add, float eps,
                               int K, float* y) {
  __shared__ double red[32];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* xm = x + (size_t)m * K;
  double ss = 0.0;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float v = xm[k];
    ss += (double)v * v;
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  double tot = 0.0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
  const float rinv = (float)(1.0 / sqrt(tot / (double)K + (double)eps));
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    float v = __fmul_rn(__fmul_rn(xm[k], rinv), gamma[k]);
    if (add) v = __fadd_rn(add[(size_t)m * K + k], v);
    y[(size_t)m * K + k] = v;
  }
}

// The same for K <= 4096, K % 4 == 0 and 16-byte aligned rows: every thread holds its (up to
// four) float4 of the row in registers, so x is read once and all loads of the launch -- x,
// gamma, the addend -- are in flight together (one memory round trip instead of two; gamma
// does not depend on the previous kernel and is fetched before the dependency wait).
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float* x, const float* gamma,
                                                          const float* add, float eps, int K,
                                                          float* y) {
  __shared__ double red[8];
  pdl_trigger();
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = K >> 2;
  float4 g[4], v[4], a[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * 256;
    g[i] = idx < nvec ? __ldg(reinterpret_cast<const float4*>(gamma) + idx)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const float4* xm = reinterpret_cast<const float4*>(x + (size_t)m * K);
  const float4* am = add ? reinterpret_cast<const float4*>(add + (size_t)m * K) : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * 256;
    v[i] = idx < nvec ? xm[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
    a[i] = (am && idx < nvec) ? am[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  double ss = 0.0;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    ss += (double)v[i].x * v[i].x + (double)v[i].y * v[i].y + (double)v[i].z * v[i].z +
          (double)v[i].w * v[i].w;
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  double tot = 0.0;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rinv = (float)(1.0 / sqrt(tot / (double)K + (double)eps));
  float4* ym = reinterpret_cast<float4*>(y + (size_t)m * K);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx >= nvec) continue;
    float4 o;
    o.x = __fmul_rn(__fmul_rn(v[i].x, rinv), g[i].x);
    o.y = __fmul_rn(__fmul_rn(v[i].y, rinv), g[i].y);
    o.z = __fmul_rn(__fmul_rn(v[i].z, rinv), g[i].z);
    o.w = __fmul_rn(__fmul_rn(v[i].w, rinv), g[i].w);
    if (am) {
      o.x = __fadd_rn(a[i].x, o.x);
      o.y = __fadd_rn(a[i].y, o.y);
      o.z = __fadd_rn(a[i].z, o.z);
      o.w = __fadd_rn(a[i].w, o.w);
    }
    ym[idx] = o;
  }
}

// ---- RoPE (NeoX pairs d, d + D/2) + f16 KV-cache write ------------------------------------

// One thread per (token, head, pair); the element's arithmetic lives in rope.cuh.
__global__ void rope_kv_kernel(const __grid_constant__ RopeParams p) {
  pdl_trigger();
  pdl_wait();
  const int per_seq = (p.H + 2 * p.Hkv) * (p.D >> 1);
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)p.B * per_seq) return;
  rope_kv_element<false>(p, idx);
}

// (cos, sin) of every (token, pair) angle of a step: [B][D/2]
__global__ void rope_table_kernel(const int32_t* pos, int B, int T, int D, double base,
                                  double2* table) {
  pdl_trigger();
  pdl_wait();
  const int half = D >> 1;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * half) return;
  const int b = idx / half, i = idx % half;
  const int cb = b / T;
  table[idx] = rope_angle(pos[cb] + (b - cb * T), i, D, base);
}

// ---- greedy argmax: first strict maximum (Hesper/Models/BitNet.lean:474-479) ---------------

// A float and its index as one ordered 64-bit key: larger value wins, then smaller index.
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // monotone map float -> uint
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - idx);
}

__global__ void argmax_kernel(const float* logits, long V, int32_t* out) {
  __shared__ unsigned long long red[32];
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = logits + (size_t)m * V;
  unsigned long long best = 0;
  for (long i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v == v) {  // NaN never wins
      const unsigned long long k = argmax_key(v, (uint32_t)i);
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
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) best = red[i] > best ? red[i] : best;
    out[m] = best ? (int32_t)(0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFull)) : 0;
  }
}

// ---- LM head: 16-bit table [V][K] x f32 activations, fused RMSNorm prologue and argmax -----

constexpr int kLMThreads = 256;
constexpr int kLMWarps = kLMThreads / 32;
constexpr int kLMRows = 2;  // rows per tile

struct LMParams {
  const uint16_t* table;  // [V][K] bf16 (dtype 0) or f16 (dtype 1)
  const float* x;         // [M][K]
  const float* gamma;     // nullable: final RMSNorm fused in front
  float* logits;          // nullable [M][V]
  unsigned long long* keys;  // [M] running argmax keys (zeroed by the caller side kernel)
  long V;
  int K, M, dtype, stages;
  float eps;
  uint32_t* status;
};

template <int MT>
__global__ void __launch_bounds__(kLMThreads, 1) lmhead_kernel(const __grid_constant__ LMParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, S = p.stages;
  const int rowbytes = K * 2;
  const int stage_bytes = kLMRows * rowbytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  size_t off = ((size_t)kLMWarps * S * 8 + 127) & ~size_t(127);
  double* red = reinterpret_cast<double*>(smem + off);
  off += 16 * 8;
  float* xs = reinterpret_cast<float*>(smem + off);  // [MT][K]
  off += (size_t)MT * K * 4;
  off = (off + 127) & ~size_t(127);
  uint8_t* wstage = smem + off + (size_t)warp * S * stage_bytes;
  uint64_t* mybar = bars + warp * S;

  const long ntiles = (p.V + kLMRows - 1) / kLMRows;
  const long t0 = (long)blockIdx.x * ntiles / gridDim.x;
  const long t1 = (long)(blockIdx.x + 1) * ntiles / gridDim.x;

  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&mybar[s], 1);
    fence_mbar_init();
  }
  __syncwarp();
  const uint64_t pol = policy_evict_first();
  int issued = 0, consumed = 0;
  long tprod = t0 + warp;
  auto produce = [&]() {
    const long row = tprod * kLMRows;
    const int nr = (int)min((long)kLMRows, p.V - row);
    if (lane == 0) {
      const int stage = issued % S;
      const uint32_t bytes = (uint32_t)nr * rowbytes;
      mbar_arrive_expect_tx(&mybar[stage], bytes);
      bulk_g2s_stream(wstage + (size_t)stage * stage_bytes,
                      reinterpret_cast<const uint8_t*>(p.table) + (size_t)row * rowbytes, bytes,
                      &mybar[stage], pol);
    }
    tprod += kLMWarps;
    ++issued;
  };
  while (issued < S && tprod < t1) produce();
  pdl_trigger();
  pdl_wait();

  for (int m0 = 0; m0 < p.M; m0 += MT) {
    __syncthreads();
    // activations (optionally RMS-normalised) of MT tokens into shared memory
    for (int mt = 0; mt < MT; ++mt) {
      const int m = m0 + mt;
      float* xm = xs + (size_t)mt * K;
      if (m >= p.M) {
        for (int k = tid; k < K; k += kLMThreads) xm[k] = 0.f;
        continue;
      }
      const float* xg = p.x + (size_t)m * K;
      float rinv = 1.f;
      if (p.gamma) {
        double ss = 0.0;
        for (int k = tid; k < K; k += kLMThreads) {
          const float v = xg[k];
          ss += (double)v * v;
        }
        ss = warp_sum(ss);
        __syncthreads();
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        ss = 0.0;
        for (int i = 0; i < kLMWarps; ++i) ss += red[i];
        rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
      }
      for (int k = tid; k < K; k += kLMThreads)
        xm[k] = p.gamma ? __fmul_rn(__fmul_rn(xg[k], rinv), p.gamma[k]) : xg[k];
    }
    __syncthreads();
    if (m0 > 0) {
      tprod = t0 + warp;
      for (int n = 0; n < S && tprod < t1; ++n) produce();
    }
    unsigned long long best[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) best[mt] = 0;

    for (long t = t0 + warp; t < t1; t += kLMWarps) {
      const int stage = consumed % S;
      mbar_wait(&mybar[stage], (uint32_t)((consumed / S) & 1), p.status);
      const uint8_t* ws = wstage + (size_t)stage * stage_bytes;
      float acc[MT][kLMRows];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < kLMRows; ++r) acc[mt][r] = 0.f;
      // lane takes 16-byte units (8 weights) lane, lane+32, ...
      for (int c = lane; c < (K >> 3); c += 32) {
        float w[kLMRows][8];
#pragma unroll
        for (int r = 0; r < kLMRows; ++r) {
          const uint4 u = *reinterpret_cast<const uint4*>(ws + r * rowbytes + c * 16);
          const uint32_t q[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (p.dtype == 0) {
              w[r][2 * j] = __uint_as_float(q[j] << 16);
              w[r][2 * j + 1] = __uint_as_float(q[j] & 0xFFFF0000u);
            } else {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&q[j]));
              w[r][2 * j] = f.x;
              w[r][2 * j + 1] = f.y;
            }
          }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const float4 xa = *reinterpret_cast<const float4*>(xs + (size_t)mt * K + c * 8);
          const float4 xb = *reinterpret_cast<const float4*>(xs + (size_t)mt * K + c * 8 + 4);
          const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
          for (int r = 0; r < kLMRows; ++r)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[mt][r] = fmaf(w[r][j], xv[j], acc[mt][r]);
        }
      }
      __syncwarp();
      if (tprod < t1) produce();
      const long row0 = t * kLMRows;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int r = 0; r < kLMRows; ++r) {
          const float v = warp_sum(acc[mt][r]);
          const long row = row0 + r;
          if (row < p.V && m0 + mt < p.M) {
            if (lane == 0 && p.logits) p.logits[(size_t)(m0 + mt) * p.V + row] = v;
            if (v == v) {
              const unsigned long long k = argmax_key(v, (uint32_t)row);
              best[mt] = k > best[mt] ? k : best[mt];
            }
          }
        }
      }
      ++consumed;
    }
    if (lane == 0 && p.keys) {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
        if (m0 + mt < p.M && best[mt]) atomicMax(&p.keys[m0 + mt], best[mt]);
    }
  }
}

// keys -> token ids; appends them to the token log and clears the keys for the next step.
__global__ void argmax_finish_kernel(unsigned long long* keys, int M, int32_t* out,
                                     int32_t* log, const int32_t* log_index, int log_stride) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  const unsigned long long k = keys[m];
  const int32_t tok = k ? (int32_t)(0xFFFFFFFFu - (uint32_t)(k & 0xFFFFFFFFull)) : 0;
  out[m] = tok;
  if (log && log_index) {
    const int li = log_index[0];
    if (li >= 0 && li < log_stride) log[(size_t)m * log_stride + li] = tok;
  }
  keys[m] = 0ull;
}

// ---- GLU epilogues --------------------------------------------------------------------

__global__ void relu2_mul_kernel(const float* g, const float* u, long n, float* y) {
  pdl_trigger();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float r = g[i] > 0.f ? g[i] : 0.f;
    y[i] = __fmul_rn(__fmul_rn(r, r), u[i]);
  }
}
__global__ void gelu_mul_kernel(const float* g, const float* u, long n, float* y) {
  pdl_trigger();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float x = g[i];
    const float t = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    y[i] = 0.5f * x * (1.0f + tanhf(t)) * u[i];
  }
}

// adds `delta` to each of n int32 counters (positions, sequence lengths, log index)
__global__ void add_i32_kernel(int32_t* a, int n, int delta) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) a[i] += delta;
}

template <int MT>
static cudaError_t lm_launch(hb200_ctx* ctx, const LMParams& p, int grid, size_t smem,
                             cudaStream_t st) {
  auto kern = lmhead_kernel<MT>;
  if (hb_func_smem(ctx, reinterpret_cast<const void*>(kern), (size_t)ctx->smem_optin) != HB200_OK)
    return cudaErrorInvalidValue;
  return launch_pdl(kern, dim3(grid), dim3(kLMThreads), smem, st, ctx->pdl, p);
}

}  // namespace hb

using namespace hb;

extern "C" int hb200_embed_lookup(hb200_ctx* ctx, const void* d_table, int dtype, long V, int K,
                                  const int32_t* d_ids, int M, float scale, float* d_y,
                                  hb200_stream stream) {
  HB_REQUIRE(ctx && d_table && d_ids && d_y, "embed: null pointer");
  HB_REQUIRE(dtype >= 0 && dtype <= 2 && V >= 1 && K >= 1 && M >= 1, "embed: bad shape or dtype");
  HB_CUDA(launch_pdl(embed_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream),
                     ctx->pdl, d_table, dtype, d_ids, K, V, scale, d_y));
  return HB200_OK;
}

extern "C" int hb200_rmsnorm(hb200_ctx* ctx, const float* d_x, const float* d_gamma,
                             const float* d_add, float eps, int M, int K, float* d_y,
                             hb200_stream stream) {
  HB_REQUIRE(ctx && d_x && d_gamma && d_y, "rmsnorm: null pointer");
  HB_REQUIRE(M >= 1 && K >= 1, "rmsnorm: M=%d K=%d", M, K);
  const uintptr_t bits = reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_gamma) |
                         reinterpret_cast<uintptr_t>(d_add) | reinterpret_cast<uintptr_t>(d_y);
  if (K % 4 == 0 && K <= 4096 && (bits & 15) == 0) {
    HB_CUDA(launch_pdl(rmsnorm_vec_kernel, dim3(M), dim3(256), 0,
                       static_cast<cudaStream_t>(stream), ctx->pdl, d_x, d_gamma, d_add, eps, K,
                       d_y));
    return HB200_OK;
  }
  HB_CUDA(launch_pdl(rmsnorm_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream),
                     ctx->pdl, d_x, d_gamma, d_add, eps, K, d_y));
  return HB200_OK;
}

static int rope_run(hb200_ctx* ctx, float* d_q, const float* d_k, const float* d_v,
                    void* d_k_cache, void* d_v_cache, const int32_t* d_pos, int nseq, int T, int H,
                    int Hkv, int D, int cache_slots, int ring, float rope_base,
                    hb200_stream stream, const double* d_table = nullptr) {
  HB_REQUIRE(ctx && d_q && d_k && d_v && d_k_cache && d_v_cache && d_pos, "rope: null pointer");
  HB_REQUIRE(nseq >= 1 && T >= 1 && (long)nseq * T < (1l << 24) && H >= 1 && Hkv >= 1 && D >= 2 &&
                 D % 2 == 0 && cache_slots >= 1,
             "rope: bad shape");
  HB_REQUIRE(!ring || T <= cache_slots, "rope: %d tokens per call into a ring of %d slots", T,
             cache_slots);
  const int B = nseq * T;
  RopeParams p = {d_q, d_k, d_v, static_cast<__half*>(d_k_cache), static_cast<__half*>(d_v_cache),
                  d_pos, B, H, Hkv, D, cache_slots, ring, T, (double)rope_base,
                  reinterpret_cast<const double2*>(d_table)};
  const long n = (long)B * (H + 2 * Hkv) * (D / 2);
  HB_CUDA(launch_pdl(rope_kv_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                     static_cast<cudaStream_t>(stream), ctx->pdl, p));
  return HB200_OK;
}

extern "C" int hb200_rope_table(hb200_ctx* ctx, const int32_t* d_pos, int B, int T, int D,
                                float rope_base, double* d_table, hb200_stream stream) {
  HB_REQUIRE(ctx && d_pos && d_table && B >= 1 && T >= 1 && D >= 2 && D % 2 == 0,
             "rope_table: bad argument");
  HB_REQUIRE((reinterpret_cast<uintptr_t>(d_table) & 15) == 0, "rope_table: table must be 16-byte aligned");
  const int n = B * T * (D / 2);
  HB_CUDA(launch_pdl(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0,
                     static_cast<cudaStream_t>(stream), ctx->pdl, d_pos, B * T, T, D,
                     (double)rope_base, reinterpret_cast<double2*>(d_table)));
  return HB200_OK;
}

extern "C" int hb200_rope_kv_write(hb200_ctx* ctx, float* d_q, const float* d_k, const float* d_v,
                                   void* d_k_cache, void* d_v_cache, const int32_t* d_pos, int B,
                                   int H, int Hkv, int D, int cache_slots, int ring,
                                   float rope_base, hb200_stream stream) {
  return rope_run(ctx, d_q, d_k, d_v, d_k_cache, d_v_cache, d_pos, B, 1, H, Hkv, D, cache_slots,
                  ring, rope_base, stream);
}

extern "C" int hb200_rope_kv_write_angles(hb200_ctx* ctx, float* d_q, const float* d_k,
                                          const float* d_v, void* d_k_cache, void* d_v_cache,
                                          const int32_t* d_pos, const double* d_table, int B,
                                          int H, int Hkv, int D, int cache_slots, int ring,
                                          hb200_stream stream) {
  HB_REQUIRE(d_table != nullptr, "rope (angles): null table");
  return rope_run(ctx, d_q, d_k, d_v, d_k_cache, d_v_cache, d_pos, B, 1, H, Hkv, D, cache_slots,
                  ring, 0.f, stream, d_table);
}

extern "C" int hb200_rope_kv_write_prefill(hb200_ctx* ctx, float* d_q, const float* d_k,
                                           const float* d_v, void* d_k_cache, void* d_v_cache,
                                           const int32_t* d_pos0, int B, int T, int H, int Hkv,
                                           int D, int cache_slots, float rope_base,
                                           hb200_stream stream) {
  return rope_run(ctx, d_q, d_k, d_v, d_k_cache, d_v_cache, d_pos0, B, T, H, Hkv, D, cache_slots, 0,
                  rope_base, stream);
}

extern "C" int hb200_rope_kv_write_prefill_angles(hb200_ctx* ctx, float* d_q, const float* d_k,
                                                  const float* d_v, void* d_k_cache,
                                                  void* d_v_cache, const int32_t* d_pos0,
                                                  const double* d_table, int B, int T, int H,
                                                  int Hkv, int D, int cache_slots, int ring,
                                                  hb200_stream stream) {
  HB_REQUIRE(d_table != nullptr, "rope (prefill, angles): null table");
  return rope_run(ctx, d_q, d_k, d_v, d_k_cache, d_v_cache, d_pos0, B, T, H, Hkv, D, cache_slots,
                  ring, 0.f, stream, d_table);
}

extern "C" int hb200_argmax(hb200_ctx* ctx, const float* d_logits, long V, int M, int32_t* d_out,
                            hb200_stream stream) {
  HB_REQUIRE(ctx && d_logits && d_out && V >= 1 && M >= 1, "argmax: bad argument");
  HB_CUDA(launch_pdl(argmax_kernel, dim3(M), dim3(1024), 0, static_cast<cudaStream_t>(stream),
                     ctx->pdl, d_logits, V, d_out));
  return HB200_OK;
}

extern "C" size_t hb200_lmhead_scratch_bytes(int M) { return (size_t)(M < 1 ? 1 : M) * 8; }

extern "C" int hb200_lmhead_argmax(hb200_ctx* ctx, const void* d_table, int dtype, long V, int K,
                                   const float* d_x, int M, const float* d_rms_gamma,
                                   float rms_eps, float* d_logits, int32_t* d_argmax,
                                   void* d_scratch, int32_t* d_token_log,
                                   const int32_t* d_log_index, int log_stride,
                                   hb200_stream stream) {
  HB_REQUIRE(ctx && d_table && d_x && d_argmax && d_scratch, "lmhead: null pointer");
  HB_REQUIRE((dtype == 0 || dtype == 1) && V >= 1 && K >= 8 && K % 8 == 0 && M >= 1 && M <= 64,
             "lmhead: bad shape or dtype (K must be a multiple of 8, M <= 64)");
  HB_REQUIRE((reinterpret_cast<uintptr_t>(d_table) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(d_x) & 15) == 0,
             "lmhead: table and x must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M >= 16 && K % 64 == 0 && !ctx->no_mma) {  // a real contraction: tensor-core path
    const int rc = hb_lmhead_mma_run(ctx, d_table, dtype, V, K, d_x, M, d_rms_gamma, rms_eps,
                                     d_logits, static_cast<unsigned long long*>(d_scratch), st);
    if (rc != HB200_OK) return rc;
    HB_CUDA(launch_pdl(argmax_finish_kernel, dim3((M + 63) / 64), dim3(64), 0, st, ctx->pdl,
                       static_cast<unsigned long long*>(d_scratch), M, d_argmax, d_token_log,
                       d_log_index, log_stride));
    return HB200_OK;
  }
  LMParams p = {};
  p.table = static_cast<const uint16_t*>(d_table);
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.logits = d_logits;
  p.keys = static_cast<unsigned long long*>(d_scratch);
  p.V = V;
  p.K = K;
  p.M = M;
  p.dtype = dtype;
  p.eps = rms_eps;
  p.status = ctx->d_status;
  const int MT = M == 1 ? 1 : (M <= 4 ? 4 : 8);
  const size_t stage = (size_t)kLMRows * K * 2;
  const size_t fixed = (((size_t)kLMWarps * 4 * 8 + 127) & ~size_t(127)) + 128 + (size_t)MT * K * 4 + 128;
  int stages = 4;
  while (stages > 1 && fixed + (size_t)kLMWarps * stages * stage > (size_t)ctx->smem_optin) --stages;
  const size_t smem = fixed + (size_t)kLMWarps * stages * stage;
  HB_REQUIRE(smem <= (size_t)ctx->smem_optin, "lmhead: K=%d does not fit shared memory", K);
  p.stages = stages;
  const long ntiles = (V + kLMRows - 1) / kLMRows;
  const int grid = ntiles < ctx->sm_count ? (int)ntiles : ctx->sm_count;
  cudaError_t e = MT == 1 ? lm_launch<1>(ctx, p, grid, smem, st)
                          : (MT == 4 ? lm_launch<4>(ctx, p, grid, smem, st)
                                     : lm_launch<8>(ctx, p, grid, smem, st));
  if (e != cudaSuccess) return cuda_fail(e, "lmhead launch");
  HB_CUDA(launch_pdl(argmax_finish_kernel, dim3((M + 63) / 64), dim3(64), 0, st, ctx->pdl,
                     static_cast<unsigned long long*>(d_scratch), M, d_argmax, d_token_log,
                     d_log_index, log_stride));
  return HB200_OK;
}

extern "C" int hb200_relu2_mul(hb200_ctx* ctx, const float* d_gate, const float* d_up, long n,
                               float* d_y, hb200_stream stream) {
  HB_REQUIRE(ctx && d_gate && d_up && d_y && n >= 1, "relu2_mul: bad argument");
  HB_CUDA(launch_pdl(relu2_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                     static_cast<cudaStream_t>(stream), ctx->pdl, d_gate, d_up, n, d_y));
  return HB200_OK;
}

extern "C" int hb200_gelu_mul(hb200_ctx* ctx, const float* d_gate, const float* d_up, long n,
                              float* d_y, hb200_stream stream) {
  HB_REQUIRE(ctx && d_gate && d_up && d_y && n >= 1, "gelu_mul: bad argument");
  HB_CUDA(launch_pdl(gelu_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                     static_cast<cudaStream_t>(stream), ctx->pdl, d_gate, d_up, n, d_y));
  return HB200_OK;
}

extern "C" int hb200_add_i32(hb200_ctx* ctx, int32_t* d_a, int n, int delta, hb200_stream stream) {
  HB_REQUIRE(ctx && d_a && n >= 1, "add_i32: bad argument");
  HB_CUDA(launch_pdl(add_i32_kernel, dim3((n + 255) / 256), dim3(256), 0,
                     static_cast<cudaStream_t>(stream), ctx->pdl, d_a, n, delta));
  return HB200_OK;
}
