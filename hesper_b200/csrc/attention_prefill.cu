// attention_prefill.cu -- causal GQA attention of a prompt chunk, tiled over queries.
//
// T new query tokens per sequence against the f16 KV cache that already holds them (the role
// of the reference's batched prefill kernels, flashAttentionBatchKernelF16 and its SWA variant,
// Hesper/WGSL/FlashAttention.lean:601,1621-1624; math of flashAttentionSpec, :60-90).  The
// decode kernel can serve a chunk by treating every token as a query of its own, but then every
// token streams its whole visible cache; here a CTA owns 64 query rows -- 64 / G consecutive
// tokens times the G query heads of one KV head -- and walks the positions those tokens see in
// tiles of 64 (32 at head_dim 256), so a K/V tile is read once per 64 / G tokens:
//   * Q (pre-multiplied by scale * log2 e, f16) stays in shared memory for the whole CTA;
//   * K/V tiles arrive by 16-byte cp.async into a two-stage ring (XOR-swizzled 16-byte units,
//     conflict-free ldmatrix); ring caches map position p to slot p % slots;
//   * S = Q K^T and O += P V on mma.sync.m16n8k16 (f16 in, f32 accumulate), one warp per 16 rows;
//     the softmax is the online form in the exp2 domain, P is rounded to f16 for the second
//     product (same rounding as the decode kernel's FAST mode: bar 2e-3 against an f64 evaluation);
//   * a row's visible positions are [max(0, pos - window + 1), pos] with pos the token's own
//     position: causal inside the chunk, sliding window if asked.
#include <math_constants.h>

#include "common.cuh"

namespace hb {

constexpr int kPfWarps = 4;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kPfRows = 64;   // query rows per CTA
// positions per K/V tile: 64, and 32 at head_dim 256, where the 128 output accumulators per
// lane leave no registers for a 64-wide score tile
template <int D>
struct PfTile {
  static constexpr int value = D >= 256 ? 32 : 64;
};

struct PfParams {
  const void* q;        // [nseq][T][H][D] f32 or f16
  const __half* k;      // [nseq][Hkv][slots][D]
  const __half* v;
  const int32_t* seqlens;  // [nseq] lengths after the T tokens
  float* out;           // [nseq][T][H][D]
  int q_is_f16;
  int nseq, T, H, Hkv, G, slots, window, ring;
  float scale_log2;
  // nsplit > 1: the K/V tiles of a query tile are dealt to nsplit CTAs (a long context at a small
  // batch would otherwise fill a fraction of the SMs); each writes its unnormalised partial and
  // its (max, sum), attn_prefill_merge_kernel combines them
  int nsplit;
  float* part_o;   // [nseq][T][H][nsplit][D]
  float* part_ml;  // [nseq][T][H][nsplit][2]  (max in the exp2 domain, sum)
};

template <int D>
struct PfCfg {
  static constexpr int kQStride = D + 8;                      // halves per Q row (bank spread)
  static constexpr int kQBytes = kPfRows * kQStride * 2;
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTile = PfTile<D>::value;
  static constexpr int kTileBytes = kTile * kRowBytes;        // one of K or V
  static constexpr int kSmem = kQBytes + 2 * 2 * kTileBytes;  // Q + two stages of (K, V)
};

__device__ __forceinline__ void pf_cp16(void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n)
               : "memory");
}
__device__ __forceinline__ void pf_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pf_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void pf_ldsm(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void pf_ldsm_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(kPfThreads, D >= 256 ? 1 : 2)
    attn_prefill_tiled_kernel(const __grid_constant__ PfParams p) {
  using Cfg = PfCfg<D>;
  constexpr int KS = D / 16;  // k-steps of the first product
  constexpr int NO = D / 8;   // n-tiles of the output
  constexpr int CPR = D / 8;  // 16-byte units per cache row
  constexpr int TILE = Cfg::kTile, NS = TILE / 8;  // positions and score n-tiles per K/V tile
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = p.G, TQ = kPfRows / G;
  const int qt = blockIdx.x / p.nsplit, split = blockIdx.x % p.nsplit;
  const int kvh = blockIdx.y, b = blockIdx.z;

  __half* qs = reinterpret_cast<__half*>(smem);
  uint8_t* stage0 = smem + Cfg::kQBytes;

  pdl_trigger();
  pdl_wait();  // q, the cache rows of this chunk and seqlens come from earlier kernels

  int len = max(p.seqlens[b], 0);  // positions after the chunk
  if (!p.ring) len = min(len, p.slots);  // a corrupt length never overruns a linear cache
  const int t0 = qt * TQ;                // first token of this CTA
  const int t1 = min(t0 + TQ, p.T) - 1;  // last one
  // positions of the chunk's tokens: token t sits at len - T + t
  const int pos_first = len - p.T + t0, pos_last = len - p.T + t1;
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, pos_first - p.window + 1);
  const int kv_hi = pos_last;  // inclusive
  const int ntiles_all = kv_hi >= kv_lo ? (kv_hi - kv_lo) / TILE + 1 : 0;
  // this CTA's share of the tiles
  const int tps = (ntiles_all + p.nsplit - 1) / p.nsplit;
  const int j0 = split * tps;
  const int ntiles = max(0, min(ntiles_all, j0 + tps) - j0);

  const __half* kbase = p.k + ((size_t)b * p.Hkv + kvh) * (size_t)p.slots * D;
  const __half* vbase = p.v + ((size_t)b * p.Hkv + kvh) * (size_t)p.slots * D;
  auto issue = [&](int j, int st) {
    uint8_t* ks = stage0 + (size_t)st * 2 * Cfg::kTileBytes;
    uint8_t* vs = ks + Cfg::kTileBytes;
    const int p0 = kv_lo + (j0 + j) * TILE;
#pragma unroll
    for (int i = 0; i < TILE * CPR / kPfThreads; ++i) {
      const int u = tid + i * kPfThreads;
      const int row = u / CPR, cc = u % CPR;
      const int pos = p0 + row;
      const bool ok = pos <= kv_hi && pos >= 0;
      int slot = ok ? pos : 0;
      if (p.ring) slot %= p.slots;
      const size_t goff = (size_t)slot * D + cc * 8;
      const int soff = row * Cfg::kRowBytes + ((cc ^ (row & 7)) << 4);
      pf_cp16(ks + soff, kbase + goff, ok);
      pf_cp16(vs + soff, vbase + goff, ok);
    }
  };
  if (ntiles > 0) issue(0, 0);
  pf_commit();

  // Q rows: row r = (token t0 + r / G, head kvh * G + r % G), scaled, f16; rows past T are zero
  for (int i = tid; i < kPfRows * (D / 4); i += kPfThreads) {
    const int r = i / (D / 4), d4 = i % (D / 4);
    const int t = t0 + r / G, h = kvh * G + r % G;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < p.T) {
      const size_t qi = (((size_t)b * p.T + t) * p.H + h) * D + 4 * d4;
      if (p.q_is_f16) {
        const __half2* hq = reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(p.q) + qi);
        const float2 a = __half22float2(hq[0]), c = __half22float2(hq[1]);
        v = make_float4(a.x, a.y, c.x, c.y);
      } else {
        v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.q) + qi);
      }
    }
    uint2 w;
    w.x = pf_pack(v.x * p.scale_log2, v.y * p.scale_log2);
    w.y = pf_pack(v.z * p.scale_log2, v.w * p.scale_log2);
    *reinterpret_cast<uint2*>(qs + r * Cfg::kQStride + 4 * d4) = w;
  }
  __syncthreads();

  // this lane's two rows (g and g + 8 of the warp's 16) and what they may see
  const int rA = 16 * warp + g, rB = rA + 8;
  const int tA = t0 + rA / G, tB = t0 + rB / G;
  const int posA = len - p.T + tA, posB = len - p.T + tB;
  const int loA = p.window > 0 ? max(0, posA - p.window + 1) : 0;
  const int loB = p.window > 0 ? max(0, posB - p.window + 1) : 0;
  const bool liveA = tA < p.T, liveB = tB < p.T;

  float mA = -CUDART_INF_F, mB = -CUDART_INF_F, lA = 0.f, lB = 0.f;
  float o[NO][4];
#pragma unroll
  for (int n = 0; n < NO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int j = 0; j < ntiles; ++j) {
    if (j + 1 < ntiles) issue(j + 1, (j + 1) & 1);
    pf_commit();
    pf_wait<1>();
    __syncthreads();  // tile j is in shared memory for every warp
    const uint8_t* ks = stage0 + (size_t)(j & 1) * 2 * Cfg::kTileBytes;
    const uint8_t* vs = ks + Cfg::kTileBytes;
    const int p0 = kv_lo + (j0 + j) * TILE;

    // ---- S = Q K^T: 16 rows x TILE positions per warp -------------------------------------
    float s[NS][4];
#pragma unroll
    for (int n = 0; n < NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      uint32_t a[4];
      {
        // A fragment of Q: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15) of this warp's 16 rows
        const int row = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int col = 16 * kk + (lane >> 4) * 8;
        pf_ldsm(a, qs + row * Cfg::kQStride + col);
      }
#pragma unroll
      for (int np = 0; np < NS / 2; ++np) {  // two n-tiles (16 positions) per ldmatrix
        uint32_t kb[4];
        // matrices: (pos 0-7, d 0-7), (pos 0-7, d 8-15), (pos 8-15, d 0-7), (pos 8-15, d 8-15)
        const int row = 16 * np + (lane & 7) + (lane >> 4) * 8;
        const int cc = 2 * kk + ((lane >> 3) & 1);
        pf_ldsm(kb, ks + row * Cfg::kRowBytes + ((cc ^ (row & 7)) << 4));
        pf_mma(s[2 * np], a, kb[0], kb[1]);
        pf_mma(s[2 * np + 1], a, kb[2], kb[3]);
      }
    }

    // ---- mask, online softmax (exp2 domain) ----------------------------------------------
    float mxA = -CUDART_INF_F, mxB = -CUDART_INF_F;
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const int pc = p0 + 8 * n + 2 * t4;
      const bool a0 = liveA && pc >= loA && pc <= posA, a1 = liveA && pc + 1 >= loA && pc + 1 <= posA;
      const bool b0 = liveB && pc >= loB && pc <= posB, b1 = liveB && pc + 1 >= loB && pc + 1 <= posB;
      s[n][0] = a0 ? s[n][0] : -CUDART_INF_F;
      s[n][1] = a1 ? s[n][1] : -CUDART_INF_F;
      s[n][2] = b0 ? s[n][2] : -CUDART_INF_F;
      s[n][3] = b1 ? s[n][3] : -CUDART_INF_F;
      mxA = fmaxf(mxA, fmaxf(s[n][0], s[n][1]));
      mxB = fmaxf(mxB, fmaxf(s[n][2], s[n][3]));
    }
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
    const float mnA = fmaxf(mA, mxA), mnB = fmaxf(mB, mxB);
    const float baseA = mnA == -CUDART_INF_F ? 0.f : mnA;  // nothing visible yet: avoid inf - inf
    const float baseB = mnB == -CUDART_INF_F ? 0.f : mnB;
    const float alA = exp2f(mA - baseA), alB = exp2f(mB - baseB);
    float sumA = 0.f, sumB = 0.f;
    uint32_t pa[NS / 2][4];  // P as A fragments of the second product: k-steps of 16 positions
#pragma unroll
    for (int n = 0; n < NS; ++n) {
      const float e0 = exp2f(s[n][0] - baseA), e1 = exp2f(s[n][1] - baseA);
      const float e2 = exp2f(s[n][2] - baseB), e3 = exp2f(s[n][3] - baseB);
      sumA += e0 + e1;
      sumB += e2 + e3;
      pa[n >> 1][(n & 1) * 2] = pf_pack(e0, e1);      // rows g
      pa[n >> 1][(n & 1) * 2 + 1] = pf_pack(e2, e3);  // rows g + 8
    }
    sumA += __shfl_xor_sync(0xffffffffu, sumA, 1);
    sumA += __shfl_xor_sync(0xffffffffu, sumA, 2);
    sumB += __shfl_xor_sync(0xffffffffu, sumB, 1);
    sumB += __shfl_xor_sync(0xffffffffu, sumB, 2);
    lA = lA * alA + sumA;
    lB = lB * alB + sumB;
    mA = mnA;
    mB = mnB;
#pragma unroll
    for (int n = 0; n < NO; ++n) {
      o[n][0] *= alA;
      o[n][1] *= alA;
      o[n][2] *= alB;
      o[n][3] *= alB;
    }

    // ---- O += P V ---------------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < NS / 2; ++kk) {  // 16 positions per step
#pragma unroll
      for (int np = 0; np < NO / 2; ++np) {  // two n-tiles (16 dims) per ldmatrix
        uint32_t vb[4];
        // transposed matrices: (pos 0-7 | 8-15) x (d 0-7 | 8-15) of this step
        const int row = 16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int cc = 2 * np + (lane >> 4);
        pf_ldsm_t(vb, vs + row * Cfg::kRowBytes + ((cc ^ (row & 7)) << 4));
        pf_mma(o[2 * np], pa[kk], vb[0], vb[1]);
        pf_mma(o[2 * np + 1], pa[kk], vb[2], vb[3]);
      }
    }
    __syncthreads();  // every warp is done with stage j & 1 before it is refilled
  }

  // ---- normalise and store, or hand the partial to the merge kernel ------------------------
  if (p.nsplit == 1) {
    const float invA = lA > 0.f ? 1.f / lA : 0.f, invB = lB > 0.f ? 1.f / lB : 0.f;
    if (liveA) {
      float* dst = p.out + (((size_t)b * p.T + tA) * p.H + kvh * G + rA % G) * D;
#pragma unroll
      for (int n = 0; n < NO; ++n)
        *reinterpret_cast<float2*>(dst + 8 * n + 2 * t4) = make_float2(o[n][0] * invA, o[n][1] * invA);
    }
    if (liveB) {
      float* dst = p.out + (((size_t)b * p.T + tB) * p.H + kvh * G + rB % G) * D;
#pragma unroll
      for (int n = 0; n < NO; ++n)
        *reinterpret_cast<float2*>(dst + 8 * n + 2 * t4) = make_float2(o[n][2] * invB, o[n][3] * invB);
    }
    return;
  }
  if (liveA) {
    const size_t pi = ((((size_t)b * p.T + tA) * p.H + kvh * G + rA % G) * p.nsplit + split);
    float* dst = p.part_o + pi * D;
#pragma unroll
    for (int n = 0; n < NO; ++n)
      *reinterpret_cast<float2*>(dst + 8 * n + 2 * t4) = make_float2(o[n][0], o[n][1]);
    if (t4 == 0) *reinterpret_cast<float2*>(p.part_ml + pi * 2) = make_float2(mA, lA);
  }
  if (liveB) {
    const size_t pi = ((((size_t)b * p.T + tB) * p.H + kvh * G + rB % G) * p.nsplit + split);
    float* dst = p.part_o + pi * D;
#pragma unroll
    for (int n = 0; n < NO; ++n)
      *reinterpret_cast<float2*>(dst + 8 * n + 2 * t4) = make_float2(o[n][2], o[n][3]);
    if (t4 == 0) *reinterpret_cast<float2*>(p.part_ml + pi * 2) = make_float2(mB, lB);
  }
}

// out = sum_s 2^(m_s - m*) O_s / sum_s 2^(m_s - m*) l_s over the splits of one (token, head).
__global__ void __launch_bounds__(128) attn_prefill_merge_kernel(const float* part_o,
                                                                 const float* part_ml, int nsplit,
                                                                 int D, float* out) {
  pdl_trigger();
  pdl_wait();
  const size_t row = blockIdx.x;  // (sequence, token, head)
  const float* ml = part_ml + row * nsplit * 2;
  float mstar = -CUDART_INF_F;
  for (int s2 = 0; s2 < nsplit; ++s2) mstar = fmaxf(mstar, __ldcg(ml + 2 * s2));
  float lsum = 0.f;
  if (mstar != -CUDART_INF_F)
    for (int s2 = 0; s2 < nsplit; ++s2) lsum += exp2f(__ldcg(ml + 2 * s2) - mstar) * __ldcg(ml + 2 * s2 + 1);
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    if (mstar != -CUDART_INF_F)
      for (int s2 = 0; s2 < nsplit; ++s2)
        acc += exp2f(__ldcg(ml + 2 * s2) - mstar) * __ldcg(part_o + (row * nsplit + s2) * D + d);
    out[row * D + d] = acc * inv;
  }
}

}  // namespace hb

using namespace hb;

// How many CTAs share the K/V range of a query tile: 1 when the query tiles alone fill the SMs,
// else enough to, but no split shorter than 4 tiles of the longest range a tile can see and
// at most 8.  A function of the shapes only (the workspace is sized with it).
static int pf_pick_splits(const hb200_ctx* ctx, int nseq, int T, int H, int Hkv, int D, int slots,
                          int window) {
  const int G = H / Hkv, TQ = kPfRows / G;
  const long ctas = (long)((T + TQ - 1) / TQ) * Hkv * nseq;
  if (ctas >= ctx->sm_count) return 1;
  const int tile = D >= 256 ? 32 : 64;
  long span = slots;
  if (window > 0 && (long)window + T < span) span = (long)window + T;
  const int tiles_max = (int)((span + tile - 1) / tile);
  int ns = (int)((ctx->sm_count + ctas - 1) / ctas);
  if (ns > 8) ns = 8;
  if (ns > tiles_max / 4) ns = tiles_max / 4;
  return ns < 1 ? 1 : ns;
}

size_t hb_attn_prefill_tiled_ws(const hb200_ctx* ctx, int nseq, int T, int H, int Hkv, int D,
                                int slots) {
  if (H % Hkv) return 0;
  const int ns = pf_pick_splits(ctx, nseq, T, H, Hkv, D, slots, 0);
  return ns > 1 ? (size_t)nseq * T * H * ns * ((size_t)D + 2) * sizeof(float) + 256 : 0;
}

// Causal attention of T query tokens per sequence on the tiled kernel.  HB200_OK when the
// launch was made, 1 when the shape is outside what it covers (the caller runs every token as a
// decode query instead), < 0 on error.
int hb_attn_prefill_tiled(hb200_ctx* ctx, const void* d_q, int q_is_f16, const void* d_k,
                          const void* d_v, const int32_t* d_seqlens, int nseq, int T, int H,
                          int Hkv, int D, int slots, int window, int ring, float scale,
                          void* d_ws, size_t ws_bytes, float* d_out, cudaStream_t st) {
  const int G = H / Hkv;
  if (!(G == 1 || G == 2 || G == 4 || G == 8)) return 1;
  if (!(D == 64 || D == 128 || D == 256)) return 1;
  if (nseq > 65535 || Hkv > 65535) return 1;
  if (q_is_f16 ? (reinterpret_cast<uintptr_t>(d_q) & 3) : (reinterpret_cast<uintptr_t>(d_q) & 15)) return 1;
  if (reinterpret_cast<uintptr_t>(d_out) & 7) return 1;
  PfParams p = {};
  p.q = d_q;
  p.k = static_cast<const __half*>(d_k);
  p.v = static_cast<const __half*>(d_v);
  p.seqlens = d_seqlens;
  p.out = d_out;
  p.q_is_f16 = q_is_f16;
  p.nseq = nseq;
  p.T = T;
  p.H = H;
  p.Hkv = Hkv;
  p.G = G;
  p.slots = slots;
  p.window = window;
  p.ring = ring;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int TQ = kPfRows / G;
  p.nsplit = pf_pick_splits(ctx, nseq, T, H, Hkv, D, slots, window);
  if (p.nsplit > 1) {
    const size_t po = (size_t)nseq * T * H * p.nsplit * (size_t)D * sizeof(float);
    const size_t need = po + (size_t)nseq * T * H * p.nsplit * 2 * sizeof(float);
    if (d_ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(d_ws) & 15)) {
      p.nsplit = 1;  // a caller's workspace sized by an older rule: one CTA per query tile
    } else {
      p.part_o = static_cast<float*>(d_ws);
      p.part_ml = reinterpret_cast<float*>(static_cast<uint8_t*>(d_ws) + po);
    }
  }
  const dim3 grid((unsigned)((T + TQ - 1) / TQ) * p.nsplit, (unsigned)Hkv, (unsigned)nseq);
  int rc;
  switch (D) {
    case 64:
      rc = hb_func_smem(ctx, reinterpret_cast<const void*>(attn_prefill_tiled_kernel<64>), PfCfg<64>::kSmem);
      if (rc) return rc;
      HB_CUDA(launch_pdl(attn_prefill_tiled_kernel<64>, grid, dim3(kPfThreads), (size_t)PfCfg<64>::kSmem,
                         st, ctx->pdl, p));
      break;
    case 128:
      rc = hb_func_smem(ctx, reinterpret_cast<const void*>(attn_prefill_tiled_kernel<128>), PfCfg<128>::kSmem);
      if (rc) return rc;
      HB_CUDA(launch_pdl(attn_prefill_tiled_kernel<128>, grid, dim3(kPfThreads),
                         (size_t)PfCfg<128>::kSmem, st, ctx->pdl, p));
      break;
    default:
      rc = hb_func_smem(ctx, reinterpret_cast<const void*>(attn_prefill_tiled_kernel<256>), PfCfg<256>::kSmem);
      if (rc) return rc;
      HB_CUDA(launch_pdl(attn_prefill_tiled_kernel<256>, grid, dim3(kPfThreads),
                         (size_t)PfCfg<256>::kSmem, st, ctx->pdl, p));
      break;
  }
  if (p.nsplit > 1)
    HB_CUDA(launch_pdl(attn_prefill_merge_kernel, dim3((unsigned)((size_t)nseq * T * H)), dim3(128), 0,
                       st, ctx->pdl, (const float*)p.part_o, (const float*)p.part_ml, p.nsplit, D,
                       d_out));
  return HB200_OK;
}
