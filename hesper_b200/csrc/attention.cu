// attention.cu -- split-K GQA decode attention over an f16 KV cache for sm_100a.
//
// What it computes: for every sequence b and query head h, softmax(scale * q.K^T) V
// over the cached positions [max(0, len - window), len), i.e. the single-head
// definition of Hesper/Training/VerifiedBackward.lean:134-142 /
// Hesper/WGSL/FlashAttention.lean:60-90 with the GQA head map of
// Hesper/WGSL/FlashAttentionExperiments.lean:71-72.  The reference's production
// kernel for this is flashAttentionVecParamsKernelV11 (+ combine) in that file
// (:45, :495, launcher :572): one workgroup per Q head, so a KV head is re-read
// by each of its Q heads, 8 splits at most, and no batch dimension.
//
// How it runs on B200:
//   * one CTA per (sequence, KV head, split): all G = H/Hkv query heads of the KV
//     head share every K/V byte read from HBM;
//   * each of the 4 warps streams its own 16-position chunks global->shared with
//     16-byte cp.async copies into an XOR-swizzled layout (conflict-free for
//     ldmatrix), 2 chunks in flight per warp, no CTA-wide barrier in the loop;
//   * scores and outputs run on the tensor cores in the transposed orientation:
//     S^T[pos,head] = K[pos,:] . Q^T and O^T[dim,head] = V^T[dim,pos] . P^T, so the
//     16 rows of an m16n8k16 MMA are all real positions / dims and the 8 columns
//     hold the query heads; P^T reaches the B-operand layout with movmatrix;
//     accumulation is f32, the online softmax works in the exp2 domain;
//   * the 4 warps merge through shared memory; with one split the CTA writes the
//     normalised output itself, otherwise it writes (max, sum, unnormalised out)
//     to the workspace and a small combine kernel merges the splits (today: the last split to
//     arrive merges them, or, for small grids, a thread-block cluster merges through the
//     leader's shared memory).
#include <math_constants.h>

#include <optional>

#include "common.cuh"

namespace hb {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kChunk = 16;       // positions per warp step
constexpr int kMaxSplits = 64;

constexpr int kMinSplitChunks = 8;  // no split shorter than 128 positions

// Splits of one (sequence, KV head) that have work at its CURRENT length: the grid is sized
// on the host for the longest sequence the cache can hold, the sequence may be much shorter.
// Returns chunks per split in `cps`; splits >= the result exit at once and are not waited for.
__device__ __forceinline__ int attn_active_splits(int nch, int nsplit, int& cps) {
  cps = (nch + nsplit - 1) / nsplit;
  if (cps < kMinSplitChunks) cps = kMinSplitChunks;
  return nch > 0 ? (nch + cps - 1) / cps : 1;
}

struct AttnParams {
  const void* q;
  const __half* k;
  const __half* v;
  const int32_t* seqlens;
  float* out;        // [B][H][D]
  float* part_out;   // [B][Hkv][nsplit][8][D]  unnormalised, f32
  float* part_meta;  // [B][Hkv][nsplit][8][2]  (max in the exp2 domain, sum)
  int q_is_f16;
  int B, H, Hkv, G, max_seq, window, nsplit;
  int T;             // query tokens per sequence (1 = decode); B counts query tokens, B/T caches
  int cluster;       // != 0: the nsplit CTAs of a (sequence, KV head) form one cluster and merge
                     // through the leader's shared memory instead of global partials + ticket
  float scale_log2;  // scale * log2(e)
  int* tickets;      // nullable: per (sequence, kv head) arrival counters, zero between calls
  int ring;          // != 0: the cache is a ring of max_seq slots, position p lives in slot
                     // p % max_seq, seqlens are true lengths (they may exceed max_seq) and the
                     // window (>= 1, window + T - 1 <= max_seq) says which positions are alive
};


// Query token b of a launch with T tokens per sequence: its cache index and how many
// positions it sees (causal: token t of the T appended ones sees all but the T-1-t last).
__device__ __forceinline__ int attn_visible_len(const AttnParams& p, int b, int& cache) {
  cache = b / p.T;
  const int t = b - cache * p.T;
  int raw = max(p.seqlens[cache], 0);
  if (!p.ring) raw = min(raw, p.max_seq);
  return max(raw - (p.T - 1 - t), 0);
}

// ---- thread-block cluster helpers (distributed shared memory) ---------------------------
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared-memory address of `local` as seen in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t cluster_map(const void* local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src),
               "r"(n)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// NS stages per warp.  D <= 128: with 3 stages two CTAs share an SM (100 KB each at D = 128),
// which hides each CTA's prologue and merge behind the other's main loop when the grid is
// several waves deep; with 4 stages a CTA has its SM alone and more chunks in flight per
// warp, which is what a grid that does not fill the GPU wants.
template <int D, int NS_ = 3>
struct AttnCfg {
  static constexpr int kStages = NS_;
  static constexpr int kRowBytes = D * 2;
  static constexpr int kTileBytes = kChunk * kRowBytes;  // one of K or V
  static constexpr int kStageBytes = 2 * kTileBytes;
  static constexpr int kQStride = D + 8;                 // halves per Q row (bank spread)
  static constexpr int kQBytes = 2 * 8 * kQStride * 2;   // Q as f16 hi and lo planes [8][D+8]
  static constexpr int kSmem = kQBytes + kAttnWarps * kStages * kStageBytes;
};

// PRECISE: the scaled query and the softmax weights are each split into two f16 terms
// (hi + lo), doubling the tensor-core work and removing their rounding from the result;
// K and V are f16 in the cache, so what remains is f32 accumulation error (~1e-6).
template <int D, bool PRECISE, int NSTAGES>
__global__ void __launch_bounds__(kAttnThreads, D >= 256 ? 1 : 2) attn_decode_kernel(const __grid_constant__ AttnParams p) {
  using Cfg = AttnCfg<D, NSTAGES>;
  constexpr int QS = Cfg::kQStride;
  constexpr int NS = Cfg::kStages;
  constexpr int CPR = D / 8;   // 16-byte chunks per row
  constexpr int KS = D / 16;   // k-steps of the score product = m-tiles of the output
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int split = blockIdx.x % p.nsplit;
  const int kvh = (blockIdx.x / p.nsplit) % p.Hkv;
  const int b = blockIdx.x / (p.nsplit * p.Hkv);
  const int G = p.G;

  __half* qs = reinterpret_cast<__half*>(smem);  // [8][D+8] hi plane, heads >= G are zero
  __half* qsl = qs + 8 * QS;                       // lo plane (PRECISE only)
  uint8_t* stage0 = smem + Cfg::kQBytes + (size_t)warp * NS * Cfg::kStageBytes;

  pdl_trigger();
  pdl_wait();  // q, the cache and seqlens come from earlier kernels of the step

  // a length outside [0, max_seq] can only come from a corrupt input: clamp, never overrun
  int cb;  // which sequence's cache
  const int len = attn_visible_len(p, b, cb);
  int start = 0;
  if (p.window > 0 && len > p.window) start = len - p.window;
  const int nch = (len - start + kChunk - 1) / kChunk;  // chunks of this sequence (<= 0 if empty)
  int cps;                                              // chunks per split
  const int nact = attn_active_splits(nch, p.nsplit, cps);
  if (split >= nact) {  // an idle split of a short sequence
    for (int i = 0; i < p.cluster; ++i) {  // the cluster's barriers still need every CTA
      cluster_arrive_release();
      cluster_wait_acquire();
    }
    return;
  }
  const int c_begin = split * cps;
  const int c_end = min(nch, c_begin + cps);

  const __half* kbase = p.k + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_seq * D;
  const __half* vbase = p.v + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_seq * D;

  // chunk c -> stage: rows of 16 positions, 16-byte units XOR-swizzled by (row & 7)
  auto issue = [&](int c, int st) {
    uint8_t* ks = stage0 + (size_t)st * Cfg::kStageBytes;
    uint8_t* vs = ks + Cfg::kTileBytes;
    const int pos0 = start + c * kChunk;
    const int slot0 = p.ring ? pos0 % p.max_seq : pos0;
#pragma unroll
    for (int i = 0; i < kChunk * CPR / 32; ++i) {
      const int qd = lane + 32 * i;
      const int row = qd / CPR, cc = qd % CPR;
      const int pos = pos0 + row;
      const bool ok = pos < len;
      int slot = slot0 + row;
      if (p.ring && slot >= p.max_seq) slot -= p.max_seq;
      const size_t goff = (size_t)(ok ? slot : 0) * D + cc * 8;
      const int soff = row * Cfg::kRowBytes + ((cc ^ (row & 7)) << 4);
      cp_async16(ks + soff, kbase + goff, ok);
      cp_async16(vs + soff, vbase + goff, ok);
    }
  };

  // prefetch this warp's first NS-1 chunks
  int cnext = c_begin + warp;
#pragma unroll
  for (int i = 0; i < NS - 1; ++i) {
    if (cnext < c_end) issue(cnext, i);
    cp_async_commit();
    cnext += kAttnWarps;
  }

  // Q -> f16, pre-multiplied by scale*log2(e), heads >= G zero
  {
    const size_t qoff = ((size_t)b * p.H + (size_t)kvh * G) * D;
    // all global loads first: interleaved with the shared-memory stores below they would
    // be issued one at a time (the compiler cannot tell the two address spaces apart)
    constexpr int QI = 8 * D / kAttnThreads;
    float qv[QI];
#pragma unroll
    for (int j = 0; j < QI; ++j) {
      const int i = tid + j * kAttnThreads;
      qv[j] = 0.f;
      if (i / D < G)
        qv[j] = p.q_is_f16 ? __half2float(reinterpret_cast<const __half*>(p.q)[qoff + i])
                           : reinterpret_cast<const float*>(p.q)[qoff + i];
    }
#pragma unroll
    for (int j = 0; j < QI; ++j) {
      const int i = tid + j * kAttnThreads;
      const int h = i / D;
      const float sv = qv[j] * p.scale_log2;
      const __half hv = __float2half_rn(sv);
      qs[h * QS + (i - h * D)] = hv;
      if (PRECISE) qsl[h * QS + (i - h * D)] = __float2half_rn(sv - __half2float(hv));
    }
  }
  __syncthreads();
  // B fragments of Q^T: head g, dims 16s+2t(+1) and 16s+2t+8(+9).  The fast path keeps
  // them in registers; the precise path re-reads hi and lo from shared memory per k-step.
  constexpr int QR = PRECISE ? 1 : KS;
  uint32_t qb[QR][2];
  if (!PRECISE) {
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      qb[s][0] = *reinterpret_cast<const uint32_t*>(qs + g * QS + 16 * s + 2 * t);
      qb[s][1] = *reinterpret_cast<const uint32_t*>(qs + g * QS + 16 * s + 2 * t + 8);
    }
  }
  auto qfrag = [&](const __half* plane, int s, uint32_t& b0, uint32_t& b1) {
    b0 = *reinterpret_cast<const uint32_t*>(plane + g * QS + 16 * s + 2 * t);
    b1 = *reinterpret_cast<const uint32_t*>(plane + g * QS + 16 * s + 2 * t + 8);
  };

  // online softmax state of heads 2t and 2t+1 (replicated over g), exp2 domain
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  float o[KS][4];  // O^T: dims 16s+g (+8), heads 2t (+1)
#pragma unroll
  for (int s = 0; s < KS; ++s) o[s][0] = o[s][1] = o[s][2] = o[s][3] = 0.f;

  int it = 0;
  for (int c = c_begin + warp; c < c_end; c += kAttnWarps, ++it) {
    // keep NS-1 chunks in flight
    if (cnext < c_end) issue(cnext, (it + NS - 1) % NS);
    cp_async_commit();
    cnext += kAttnWarps;
    cp_async_wait<NS - 1>();
    __syncwarp();

    const uint8_t* ks = stage0 + (size_t)(it % NS) * Cfg::kStageBytes;
    const uint8_t* vs = ks + Cfg::kTileBytes;

    // ---- S^T = K . Q^T : two accumulation chains to shorten the dependency ----
    float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int row = lane & 15, hi = lane >> 4;
      const uint8_t* rbase = ks + row * Cfg::kRowBytes;
#pragma unroll
      for (int s = 0; s < KS; s += 2) {
        uint32_t a[4], b0, b1;
        ldsm_x4(a, rbase + (((2 * s + hi) ^ (row & 7)) << 4));
        if (PRECISE) {
          qfrag(qs, s, b0, b1);
          mma16816(sa, a, b0, b1);
          qfrag(qsl, s, b0, b1);
          mma16816(sa, a, b0, b1);
        } else {
          mma16816(sa, a, qb[s][0], qb[s][1]);
        }
        ldsm_x4(a, rbase + (((2 * s + 2 + hi) ^ (row & 7)) << 4));
        if (PRECISE) {
          qfrag(qs, s + 1, b0, b1);
          mma16816(sb, a, b0, b1);
          qfrag(qsl, s + 1, b0, b1);
          mma16816(sb, a, b0, b1);
        } else {
          mma16816(sb, a, qb[s + 1][0], qb[s + 1][1]);
        }
      }
    }
    const int pos0 = start + c * kChunk;
    const bool v0 = pos0 + g < len, v1 = pos0 + g + 8 < len;
    const float s00 = v0 ? sa[0] + sb[0] : -CUDART_INF_F;  // (pos g,   head 2t)
    const float s01 = v0 ? sa[1] + sb[1] : -CUDART_INF_F;  // (pos g,   head 2t+1)
    const float s10 = v1 ? sa[2] + sb[2] : -CUDART_INF_F;  // (pos g+8, head 2t)
    const float s11 = v1 ? sa[3] + sb[3] : -CUDART_INF_F;  // (pos g+8, head 2t+1)

    // ---- online softmax over the 16 positions (over g: lane bits 2..4) ---------
    float mx0 = fmaxf(s00, s10), mx1 = fmaxf(s01, s11);
#pragma unroll
    for (int o_ = 4; o_ < 32; o_ <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o_));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o_));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float base0 = mn0 == -CUDART_INF_F ? 0.f : mn0;  // nothing valid yet: avoid inf-inf
    const float base1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
    const float al0 = exp2f(m0 - base0), al1 = exp2f(m1 - base1);
    const float p00 = exp2f(s00 - base0), p01 = exp2f(s01 - base1);
    const float p10 = exp2f(s10 - base0), p11 = exp2f(s11 - base1);
    float sum0 = p00 + p10, sum1 = p01 + p11;
#pragma unroll
    for (int o_ = 4; o_ < 32; o_ <<= 1) {
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, o_);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, o_);
    }
    l0 = l0 * al0 + sum0;
    l1 = l1 * al1 + sum1;
    m0 = mn0;
    m1 = mn1;

    // P^T into the B-operand layout: (pos 2t,2t+1 | head g) and (pos 2t+8,2t+9 | head g)
    const uint32_t ph0 = pack_h2(p00, p01), ph1 = pack_h2(p10, p11);
    const uint32_t pb0 = movmatrix_t(ph0);
    const uint32_t pb1 = movmatrix_t(ph1);
    uint32_t pl0 = 0, pl1 = 0;
    if (PRECISE) {  // what f16 rounding dropped from the softmax weights
      const float2 r0 = __half22float2(*reinterpret_cast<const __half2*>(&ph0));
      const float2 r1 = __half22float2(*reinterpret_cast<const __half2*>(&ph1));
      pl0 = movmatrix_t(pack_h2(p00 - r0.x, p01 - r0.y));
      pl1 = movmatrix_t(pack_h2(p10 - r1.x, p11 - r1.y));
    }

    // ---- O^T = O^T*alpha + V^T . P^T ---------------------------------------------
    {
      const int mi = lane >> 3;
      const int row = (lane & 7) + ((mi >> 1) << 3);
      const uint8_t* rbase = vs + row * Cfg::kRowBytes;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        uint32_t a[4];
        ldsm_x4_t(a, rbase + (((2 * s + (mi & 1)) ^ (row & 7)) << 4));
        o[s][0] *= al0;
        o[s][1] *= al1;
        o[s][2] *= al0;
        o[s][3] *= al1;
        mma16816(o[s], a, pb0, pb1);
        if (PRECISE) mma16816(o[s], a, pl0, pl1);
      }
    }
    __syncwarp();  // the stage may be refilled by the next iteration's copies
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its stages: reuse them for the merge

  // ---- merge the 4 warps ---------------------------------------------------------
  float* mo = reinterpret_cast<float*>(smem + Cfg::kQBytes);  // [warps][8 heads][D]
  float* mm = mo + kAttnWarps * 8 * D;                         // [warps][8][2]
#pragma unroll
  for (int s = 0; s < KS; ++s) {
    float* base = mo + (size_t)warp * 8 * D;
    base[(2 * t) * D + 16 * s + g] = o[s][0];
    base[(2 * t + 1) * D + 16 * s + g] = o[s][1];
    base[(2 * t) * D + 16 * s + g + 8] = o[s][2];
    base[(2 * t + 1) * D + 16 * s + g + 8] = o[s][3];
  }
  if (g == 0) {
    float* mb = mm + (size_t)warp * 16;
    mb[(2 * t) * 2] = m0;
    mb[(2 * t) * 2 + 1] = l0;
    mb[(2 * t + 1) * 2] = m1;
    mb[(2 * t + 1) * 2 + 1] = l1;
  }
  __syncthreads();
  bool cluster_synced = false;
  for (int i = tid; i < G * D; i += kAttnThreads) {
    const int h = i / D, d = i % D;
    float mstar = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mstar = fmaxf(mstar, mm[w * 16 + h * 2]);
    float acc = 0.f, lsum = 0.f;
    if (mstar != -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < kAttnWarps; ++w) {
        const float wgt = exp2f(mm[w * 16 + h * 2] - mstar);
        acc += wgt * mo[((size_t)w * 8 + h) * D + d];
        lsum += wgt * mm[w * 16 + h * 2 + 1];
      }
    }
    if (nact == 1) {
      p.out[((size_t)b * p.H + (size_t)kvh * G + h) * D + d] = lsum > 0.f ? acc / lsum : 0.f;
    } else if (p.cluster) {
      // into the leader's (split 0) shared memory: [split][8][D] partials, then [split][8][2]
      // (max, sum).  cluster == 1: a region of its own behind the stages.  cluster == 2 (no
      // room for that): the stage region itself, once every CTA of the cluster is past its
      // main loop and its own merge reads -- one more cluster barrier.
      if (p.cluster == 2 && !cluster_synced) {
        cluster_arrive_release();
        cluster_wait_acquire();
        cluster_synced = true;
      }
      float* cp = p.cluster == 1 ? reinterpret_cast<float*>(smem + Cfg::kSmem)
                                 : mm + kAttnWarps * 16;  // past this CTA's own merge arrays
      st_cluster_f32(cluster_map(cp + ((size_t)split * 8 + h) * D + d, 0), acc);
      if (d == 0) {
        float* cm = cp + (size_t)p.nsplit * 8 * D + ((size_t)split * 8 + h) * 2;
        st_cluster_f32(cluster_map(cm, 0), mstar);
        st_cluster_f32(cluster_map(cm + 1, 0), lsum);
      }
    } else {
      const size_t pi = (((size_t)b * p.Hkv + kvh) * p.nsplit + split) * 8 + h;
      p.part_out[pi * D + d] = acc;
      if (d == 0) {
        p.part_meta[pi * 2] = mstar;
        p.part_meta[pi * 2 + 1] = lsum;
      }
    }
  }
  if (p.cluster) {
    if (p.cluster == 2 && !cluster_synced) {  // nact == 1: the first barrier was not reached above
      cluster_arrive_release();
      cluster_wait_acquire();
    }
    // cluster barrier: every split's partial has landed in the leader's shared memory
    cluster_arrive_release();
    cluster_wait_acquire();
    if (split != 0 || nact == 1) return;
    const float* cp = p.cluster == 1
                          ? reinterpret_cast<const float*>(smem + Cfg::kSmem)
                          : mm + kAttnWarps * 16;
    const float* cm = cp + (size_t)p.nsplit * 8 * D;
    float* cw = reinterpret_cast<float*>(smem + Cfg::kQBytes);  // [nsplit][8] weights, then [8] sums
    float* cl = cw + kMaxSplits * 8;
    if (tid < 8) {
      float mstar = -CUDART_INF_F;
      for (int sidx = 0; sidx < nact; ++sidx) mstar = fmaxf(mstar, cm[(sidx * 8 + tid) * 2]);
      float lsum = 0.f;
      for (int sidx = 0; sidx < nact; ++sidx) {
        const float wgt =
            mstar == -CUDART_INF_F ? 0.f : exp2f(cm[(sidx * 8 + tid) * 2] - mstar);
        lsum += wgt * cm[(sidx * 8 + tid) * 2 + 1];
        cw[sidx * 8 + tid] = wgt;
      }
      cl[tid] = lsum;
    }
    __syncthreads();
    for (int i = tid; i < G * D / 4; i += kAttnThreads) {
      const int h = (i * 4) / D, d = (i * 4) % D;
      const float4* src = reinterpret_cast<const float4*>(cp + (size_t)h * D + d);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sidx = 0; sidx < nact; ++sidx) {
        const float4 v = src[(size_t)sidx * 2 * D];  // next split: 8*D floats further
        const float wgt = cw[sidx * 8 + h];
        acc.x = fmaf(wgt, v.x, acc.x);
        acc.y = fmaf(wgt, v.y, acc.y);
        acc.z = fmaf(wgt, v.z, acc.z);
        acc.w = fmaf(wgt, v.w, acc.w);
      }
      const float lsum = cl[h];
      const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
      float4* dst = reinterpret_cast<float4*>(p.out + ((size_t)b * p.H + (size_t)kvh * G + h) * D + d);
      *dst = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    }
    return;
  }
  if (nact == 1 || p.tickets == nullptr) return;

  // ---- the last split to finish merges all splits of its (sequence, kv head) ------------
  // Each CTA publishes its partials, then takes a ticket; whoever draws the last one knows
  // every other CTA's partials are visible (fence before the ticket, fence after) and does
  // the work the separate combine kernel would do, saving that launch.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int t = atomicAdd(&p.tickets[b * p.Hkv + kvh], 1);
    s_last = (t == nact - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float* cw = reinterpret_cast<float*>(smem + Cfg::kQBytes);  // [nsplit][8] weights, then [8] sums
  float* cl = cw + kMaxSplits * 8;
  const size_t base = ((size_t)b * p.Hkv + kvh) * p.nsplit;
  for (int i = tid; i < nact * 8; i += kAttnThreads) {  // stage (max, sum) of every split
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_meta) + base * 8 + i);
    cw[i] = ml.x;
    cw[kMaxSplits * 8 + 8 + i] = ml.y;
  }
  __syncthreads();
  if (tid < 8) {
    float mstar = -CUDART_INF_F;
    for (int sidx = 0; sidx < nact; ++sidx) mstar = fmaxf(mstar, cw[sidx * 8 + tid]);
    float lsum = 0.f;
    for (int sidx = 0; sidx < nact; ++sidx) {
      const float wgt = mstar == -CUDART_INF_F ? 0.f : exp2f(cw[sidx * 8 + tid] - mstar);
      lsum += wgt * cw[kMaxSplits * 8 + 8 + sidx * 8 + tid];
      cw[sidx * 8 + tid] = wgt;
    }
    cl[tid] = lsum;
  }
  __syncthreads();
  // 4 consecutive dims per thread, 8 splits' loads in flight at a time
  for (int i = tid; i < G * D / 4; i += kAttnThreads) {
    const int h = (i * 4) / D, d = (i * 4) % D;
    const float4* src = reinterpret_cast<const float4*>(p.part_out + (base * 8 + h) * D + d);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sidx = 0; sidx < nact; ++sidx) {
      const float4 v = __ldcg(src + (size_t)sidx * 2 * D);  // next split: 8*D floats further
      const float wgt = cw[sidx * 8 + h];
      acc.x = fmaf(wgt, v.x, acc.x);
      acc.y = fmaf(wgt, v.y, acc.y);
      acc.z = fmaf(wgt, v.z, acc.z);
      acc.w = fmaf(wgt, v.w, acc.w);
    }
    const float lsum = cl[h];
    const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
    float4* dst = reinterpret_cast<float4*>(p.out + ((size_t)b * p.H + (size_t)kvh * G + h) * D + d);
    *dst = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
  }
  if (tid == 0) p.tickets[b * p.Hkv + kvh] = 0;  // ready for the next call
}

// Merges the split partials: out = sum_s 2^(m_s - m*) O_s / sum_s 2^(m_s - m*) l_s.
// Same role as flashAttentionVecCombineKernel (Hesper/WGSL/FlashAttentionExperiments.lean:495).
__global__ void attn_combine_kernel(const __grid_constant__ AttnParams p, int D) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x % p.G;
  const int kvh = (blockIdx.x / p.G) % p.Hkv;
  const int b = blockIdx.x / (p.G * p.Hkv);
  const size_t base = ((size_t)b * p.Hkv + kvh) * p.nsplit;
  // the same active-split count as the main kernel derived; a single active split wrote
  // its result straight to `out`
  int cb;
  const int len = attn_visible_len(p, b, cb);
  int start = 0;
  if (p.window > 0 && len > p.window) start = len - p.window;
  int cps;
  const int nact = attn_active_splits((len - start + kChunk - 1) / kChunk, p.nsplit, cps);
  if (nact == 1) return;
  float mstar = -CUDART_INF_F;
  for (int s = 0; s < nact; ++s) mstar = fmaxf(mstar, p.part_meta[((base + s) * 8 + h) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, lsum = 0.f;
    if (mstar != -CUDART_INF_F) {
      for (int s = 0; s < nact; ++s) {
        const size_t pi = (base + s) * 8 + h;
        const float wgt = exp2f(p.part_meta[pi * 2] - mstar);
        acc += wgt * p.part_out[pi * D + d];
        lsum += wgt * p.part_meta[pi * 2 + 1];
      }
    }
    p.out[((size_t)b * p.H + (size_t)kvh * p.G + h) * D + d] = lsum > 0.f ? acc / lsum : 0.f;
  }
}


// ---- bit-reproducible attention (parity mode) -------------------------------------------
//
// A 30-layer network that re-quantises its activations to int8 after every block is
// chaotic at the level of its quantisation noise: one activation that rounds the other way
// because attention differed by 1e-6 grows into per-cent logit noise a few layers later.
// Comparing greedy tokens with a CPU model therefore needs an attention whose every f32
// operation and its order are specified.  This kernel is that specification (a CPU
// restatement follows it operation for operation); it is slow on purpose, never the default:
//   one warp per (sequence, query head), positions strictly in order;
//   lane i owns dims [i*D/32, (i+1)*D/32): partial = fma(q_d, k_d, partial), d ascending;
//   the 32 partials are summed by the xor-butterfly 16, 8, 4, 2, 1;
//   s = total * (scale*log2e);  online softmax with exp2_det below;
//   acc_d = fma(p, v_d, acc_d * alpha);  l = fma(l, alpha, p);  out_d = acc_d / l.
__host__ __device__ __forceinline__ float exp2_det(float x) {
  // 2^x for x <= 0 from IEEE f32 operations only: x = n + f, |f| <= 1/2, degree-6 polynomial
  if (!(x > -120.0f)) return 0.0f;
  const float n = rintf(x);
  const float f = x - n;
  float p = 1.5403530e-4f;
  p = fmaf(p, f, 1.3398874e-3f);
  p = fmaf(p, f, 9.6184370e-3f);
  p = fmaf(p, f, 5.5503324e-2f);
  p = fmaf(p, f, 2.4022648e-1f);
  p = fmaf(p, f, 6.9314720e-1f);
  p = fmaf(p, f, 1.0f);
  return ldexpf(p, (int)n);
}

template <int D>
__global__ void __launch_bounds__(32) attn_exact_kernel(const __grid_constant__ AttnParams p) {
  constexpr int DL = D / 32;
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x;
  const int h = blockIdx.x % p.H, b = blockIdx.x / p.H;
  const int kvh = h / p.G;
  int cb;
  const int len = attn_visible_len(p, b, cb);
  int start = 0;
  if (p.window > 0 && len > p.window) start = len - p.window;
  float q[DL], acc[DL];
#pragma unroll
  for (int j = 0; j < DL; ++j) {
    const size_t qi = ((size_t)b * p.H + h) * D + lane * DL + j;
    q[j] = p.q_is_f16 ? __half2float(reinterpret_cast<const __half*>(p.q)[qi])
                      : reinterpret_cast<const float*>(p.q)[qi];
    acc[j] = 0.f;
  }
  const __half* kb = p.k + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_seq * D + lane * DL;
  const __half* vb = p.v + ((size_t)cb * p.Hkv + kvh) * (size_t)p.max_seq * D + lane * DL;
  float m = -CUDART_INF_F, l = 0.f;
  for (int ps = start; ps < len; ++ps) {
    const int s = p.ring ? ps % p.max_seq : ps;  // slot of position ps
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < DL; ++j) part = fmaf(q[j], __half2float(kb[(size_t)s * D + j]), part);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    const float sc = __fmul_rn(part, p.scale_log2);
    const float mn = fmaxf(m, sc);
    const float alpha = exp2_det(__fsub_rn(m, mn));  // m = -inf: exp2_det(-inf) = 0
    const float pw = exp2_det(__fsub_rn(sc, mn));
    l = fmaf(l, alpha, pw);
#pragma unroll
    for (int j = 0; j < DL; ++j)
      acc[j] = fmaf(pw, __half2float(vb[(size_t)s * D + j]), __fmul_rn(acc[j], alpha));
    m = mn;
  }
#pragma unroll
  for (int j = 0; j < DL; ++j)
    p.out[((size_t)b * p.H + h) * D + lane * DL + j] = l > 0.f ? __fdiv_rn(acc[j], l) : 0.f;
}

// Splits per (sequence, KV head): enough CTAs for two waves over the SMs, but
// no split shorter than 8 chunks (128 positions) and at most kMaxSplits.
static int attn_pick_splits(const hb200_ctx* ctx, int B, int Hkv, int D, int max_len) {
  const long pairs = (long)B * Hkv;
  const int chunks = (max_len + kChunk - 1) / kChunk;
  // two waves of resident CTAs (measured best over the batch x length sweeps); at D <= 128
  // two CTAs share an SM
  const long resident = (long)ctx->sm_count * (D <= 128 ? 2 : 1);
  long want = (2 * resident + pairs - 1) / pairs;
  long cap = chunks / 8;
  if (cap < 1) cap = 1;
  if (want > cap) want = cap;
  if (want > kMaxSplits) want = kMaxSplits;
  if (want < 1) want = 1;
  return (int)want;
}

template <int D, bool PRECISE, int NSTAGES>
static int attn_launch_ns(hb200_ctx* ctx, const AttnParams& p, cudaStream_t st);

template <int D, bool PRECISE>
static int attn_launch(hb200_ctx* ctx, const AttnParams& p, cudaStream_t st) {
  // a grid of more than two waves of single CTAs: share the SMs (3 stages); else 4 stages
  const int grid = p.B * p.Hkv * p.nsplit;
  if constexpr (D >= 256) {
    return attn_launch_ns<D, PRECISE, 3>(ctx, p, st);  // 4 stages would not fit at this size
  } else {
    if (grid > 2 * ctx->sm_count) return attn_launch_ns<D, PRECISE, 3>(ctx, p, st);
    return attn_launch_ns<D, PRECISE, 4>(ctx, p, st);
  }
}

template <int D, bool PRECISE, int NSTAGES>
static int attn_launch_ns(hb200_ctx* ctx, const AttnParams& p, cudaStream_t st) {
  using Cfg = AttnCfg<D, NSTAGES>;
  auto kern = attn_decode_kernel<D, PRECISE, NSTAGES>;
  {
    const int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(kern), (size_t)Cfg::kSmem);
    if (rc != HB200_OK) return rc;
  }
  const int grid = p.B * p.Hkv * p.nsplit;
  if (p.cluster) {
    // the splits of one (sequence, KV head) as one cluster; partials in the leader's shared
    // memory behind the stages.  Falls back to the ticket path if the launch is refused.
    const size_t smem = (size_t)Cfg::kSmem +
                        (p.cluster == 1 ? (size_t)p.nsplit * 8 * (D + 2) * sizeof(float) : 0);
    // per context: which cluster sizes the driver would not launch, and whether this kernel
    // was already allowed non-portable cluster sizes there
    uint32_t& refused = ctx->attn_cluster_refused;
    if (!(refused >> p.nsplit & 1u) && smem <= (size_t)ctx->smem_optin) {
      cudaError_t e = cudaSuccess;
      if (hb_func_smem(ctx, reinterpret_cast<const void*>(kern), smem) != HB200_OK)
        e = cudaErrorInvalidValue;
      if (e == cudaSuccess && !hb_func_flag(ctx, reinterpret_cast<const void*>(kern))) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e == cudaSuccess) hb_func_set_flag(ctx, reinterpret_cast<const void*>(kern));
      }
      if (e == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kAttnThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)p.nsplit;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        e = cudaLaunchKernelEx(&cfg, kern, p);
      }
      if (e == cudaSuccess) return HB200_OK;
      cudaGetLastError();  // a refused launch leaves no sticky error; clear the last-error slot
      refused |= 1u << p.nsplit;
    }
    AttnParams q = p;  // ticket path
    q.cluster = 0;
    return attn_launch_ns<D, PRECISE, NSTAGES>(ctx, q, st);
  }
  HB_CUDA(launch_pdl(kern, dim3(grid), dim3(kAttnThreads), (size_t)Cfg::kSmem, st, ctx->pdl, p));
  if (p.nsplit > 1 && p.tickets == nullptr) {
    HB_CUDA(launch_pdl(attn_combine_kernel, dim3(p.B * p.H), dim3(D >= 128 ? 128 : 64), 0, st,
                       ctx->pdl, p, D));
  }
  return HB200_OK;
}

}  // namespace hb

using namespace hb;


extern "C" size_t hb200_attn_workspace_bytes(const hb200_ctx* ctx, int B, int H, int Hkv, int D,
                                             int max_seq) {
  if (!ctx || B < 1 || Hkv < 1 || D < 1) return 0;
  (void)H;
  const int ns = attn_pick_splits(ctx, B, Hkv, D, max_seq);
  if (ns == 1) return 256;  // a single split writes its result directly: nothing to stage
  return (size_t)B * Hkv * ns * 8 * ((size_t)D + 2) * sizeof(float) + 256;
}

// Decode (T = 1) and causal prefill (T > 1) share everything: a prefill token is a query with
// its own visible length over its sequence's cache.  nseq sequences, T query tokens each.
static int attn_run(hb200_ctx* ctx, const void* d_q, int q_is_f16, const void* d_k,
                    const void* d_v, const int32_t* d_seqlens, int nseq, int T, int H, int Hkv,
                    int D, int max_seq, int window, float scale, void* d_workspace,
                    size_t workspace_bytes, float* d_out, hb200_stream stream, int ring = 0) {
  HB_REQUIRE(ctx != nullptr, "attn: null context");
  HB_REQUIRE(d_q && d_k && d_v && d_seqlens && d_out, "attn: null pointer");
  HB_REQUIRE(nseq >= 1 && T >= 1 && (long)nseq * T < (1l << 24), "attn: B=%d T=%d", nseq, T);
  const int B = nseq * T;  // query tokens
  HB_REQUIRE(B >= 1 && H >= 1 && Hkv >= 1 && H % Hkv == 0, "attn: B=%d H=%d Hkv=%d", B, H, Hkv);
  const int G = H / Hkv;
  HB_REQUIRE(G <= 8, "attn: %d query heads per KV head (at most 8)", G);
  HB_REQUIRE(D == 32 || D == 64 || D == 128 || D == 256, "attn: head_dim %d not in {32,64,128,256}", D);
  HB_REQUIRE(max_seq >= 1 && window >= 0, "attn: max_seq=%d window=%d", max_seq, window);
  HB_REQUIRE(!ring || (window >= 1 && (long)window + T - 1 <= max_seq),
             "attn (ring): window %d + %d query tokens - 1 must fit the %d slots", window, T, max_seq);
  HB_REQUIRE(((reinterpret_cast<uintptr_t>(d_k) | reinterpret_cast<uintptr_t>(d_v)) & 15) == 0,
             "attn: K/V cache must be 16-byte aligned");
  // a prompt chunk in the default mode: queries tiled over tokens, each K/V tile read once per
  // 64 / G tokens (attention_prefill.cu); PRECISE / EXACT keep one decode query per token
  if (T >= 8 && D != 32 && ctx->attn_mode == HB200_ATTN_FAST) {
    const int rc = hb_attn_prefill_tiled(ctx, d_q, q_is_f16, d_k, d_v, d_seqlens, nseq, T, H, Hkv,
                                         D, max_seq, window, ring, scale, d_workspace,
                                         workspace_bytes, d_out,
                                         static_cast<cudaStream_t>(stream));
    if (rc <= 0) return rc;
  }
  AttnParams p = {};
  p.q = d_q;
  p.k = static_cast<const __half*>(d_k);
  p.v = static_cast<const __half*>(d_v);
  p.seqlens = d_seqlens;
  p.out = d_out;
  p.q_is_f16 = q_is_f16;
  p.B = B;
  p.H = H;
  p.Hkv = Hkv;
  p.G = G;
  p.max_seq = max_seq;
  p.window = window;
  p.T = T;
  p.ring = ring;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int eff_len = (window > 0 && window < max_seq) ? window : max_seq;
  p.nsplit = D == 32 ? 1 : attn_pick_splits(ctx, B, Hkv, D, eff_len);
  // Small grids (the latency-bound case) merge their splits inside a thread-block cluster of
  // at most 16 splits.
  // Beyond 16 splits the cluster would have to shorten the split list; that still wins while a
  // split stays short (<= 48 chunks of 16 positions), measured: 8000 positions in 16 splits +
  // cluster 12.9 us against 62 splits + ticket 17.6 us, 32768 positions 30.8 against 20.0 us.
  const bool short_splits = p.nsplit <= 16 || (eff_len + kChunk - 1) / kChunk <= 16 * 48;
  if (p.nsplit > 1 && short_splits &&
      (long)B * Hkv * (p.nsplit < 16 ? p.nsplit : 16) <= 2L * ctx->sm_count &&
      ctx->attn_mode != HB200_ATTN_EXACT) {
    if (p.nsplit > 16) p.nsplit = 16;
    p.cluster = D <= 128 ? 1 : 2;  // D = 256: the partials reuse the stage region (2 barriers)
  }
  if (p.nsplit > 1) {
    const size_t po = (size_t)B * Hkv * p.nsplit * 8 * (size_t)D * sizeof(float);
    const size_t need = po + (size_t)B * Hkv * p.nsplit * 8 * 2 * sizeof(float);
    HB_REQUIRE(d_workspace != nullptr && workspace_bytes >= need,
               "attn: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    HB_REQUIRE((reinterpret_cast<uintptr_t>(d_workspace) & 15) == 0,
               "attn: workspace must be 16-byte aligned");
    p.part_out = static_cast<float*>(d_workspace);
    p.part_meta = reinterpret_cast<float*>(static_cast<uint8_t*>(d_workspace) + po);
    // arrival counters live in the context (zeroed at creation, left zero by every call);
    // beyond their capacity the separate combine kernel is used instead
    p.tickets = (B * Hkv <= hb::kCtxTickets) ? ctx->d_tickets : nullptr;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the arrival counters are the context's: calls on two streams must not interleave on them
  std::optional<ScratchUse> use;
  if (p.tickets && !p.cluster) use.emplace(ctx, st);
  // head_dim 32 (the reference's smallest golden case, a debugging size) is below the MMA
  // kernel's tile: it always takes the one-warp-per-head kernel
  if (ctx->attn_mode == HB200_ATTN_EXACT || D == 32) {
    const dim3 grid(B * H);
    switch (D) {
      case 32: HB_CUDA(launch_pdl(attn_exact_kernel<32>, grid, dim3(32), 0, st, ctx->pdl, p)); break;
      case 64: HB_CUDA(launch_pdl(attn_exact_kernel<64>, grid, dim3(32), 0, st, ctx->pdl, p)); break;
      case 128: HB_CUDA(launch_pdl(attn_exact_kernel<128>, grid, dim3(32), 0, st, ctx->pdl, p)); break;
      default: HB_CUDA(launch_pdl(attn_exact_kernel<256>, grid, dim3(32), 0, st, ctx->pdl, p)); break;
    }
    return HB200_OK;
  }
  if (ctx->attn_mode == HB200_ATTN_PRECISE) {
    switch (D) {
      case 64: return attn_launch<64, true>(ctx, p, st);
      case 128: return attn_launch<128, true>(ctx, p, st);
      default: return attn_launch<256, true>(ctx, p, st);
    }
  }
  switch (D) {
    case 64: return attn_launch<64, false>(ctx, p, st);
    case 128: return attn_launch<128, false>(ctx, p, st);
    default: return attn_launch<256, false>(ctx, p, st);
  }
}

extern "C" int hb200_attn_decode(hb200_ctx* ctx, const void* d_q, int q_is_f16, const void* d_k,
                                 const void* d_v, const int32_t* d_seqlens, int B, int H, int Hkv,
                                 int D, int max_seq, int window, float scale, void* d_workspace,
                                 size_t workspace_bytes, float* d_out, hb200_stream stream) {
  return attn_run(ctx, d_q, q_is_f16, d_k, d_v, d_seqlens, B, 1, H, Hkv, D, max_seq, window, scale,
                  d_workspace, workspace_bytes, d_out, stream);
}

extern "C" size_t hb200_attn_prefill_workspace_bytes(const hb200_ctx* ctx, int B, int T, int H,
                                                     int Hkv, int D, int max_seq) {
  if (!ctx || T < 1 || B < 1 || Hkv < 1 || (long)B * T >= (1l << 24)) return 0;
  // the larger of what the two routes want: one decode query per token, or the tiled kernel
  // with the positions of a query tile split over several CTAs
  const size_t a = hb200_attn_workspace_bytes(ctx, B * T, H, Hkv, D, max_seq);
  const size_t t = hb_attn_prefill_tiled_ws(ctx, B, T, H, Hkv, D, max_seq);
  return a > t ? a : t;
}

extern "C" int hb200_attn_prefill(hb200_ctx* ctx, const void* d_q, int q_is_f16, const void* d_k,
                                  const void* d_v, const int32_t* d_seqlens, int B, int T, int H,
                                  int Hkv, int D, int max_seq, int window, float scale,
                                  void* d_workspace, size_t workspace_bytes, float* d_out,
                                  hb200_stream stream) {
  return attn_run(ctx, d_q, q_is_f16, d_k, d_v, d_seqlens, B, T, H, Hkv, D, max_seq, window, scale,
                  d_workspace, workspace_bytes, d_out, stream);
}

extern "C" int hb200_attn_ring(hb200_ctx* ctx, const void* d_q, int q_is_f16, const void* d_k,
                               const void* d_v, const int32_t* d_seqlens, int B, int T, int H,
                               int Hkv, int D, int slots, int window, float scale,
                               void* d_workspace, size_t workspace_bytes, float* d_out,
                               hb200_stream stream) {
  return attn_run(ctx, d_q, q_is_f16, d_k, d_v, d_seqlens, B, T, H, Hkv, D, slots, window, scale,
                  d_workspace, workspace_bytes, d_out, stream, 1);
}

// ---- the same operator for callers that must not allocate -----------------------------
//
// Split-K partials need scratch memory.  hb200_attn_decode takes it from the caller; this
// variant keeps it inside the library image instead, as one fixed array in device global
// memory.  Every GPU that loads the library carries those 8 MiB until the process exits.
static __device__ __align__(256) unsigned char g_attn_static_scratch[HB200_ATTN_STATIC_SCRATCH_BYTES];

// In host code the array's name is only a handle for the runtime, never a pointer a kernel
// could use: its device address is looked up once per context (hence at least once per device,
// with that device current) and kept in the context.

extern "C" int hb200_attn_decode_static(hb200_ctx* ctx, const void* d_q, int q_is_f16,
                                        const void* d_k, const void* d_v,
                                        const int32_t* d_seqlens, int B, int H, int Hkv, int D,
                                        int max_seq, int window, float scale, float* d_out,
                                        hb200_stream stream) {
  HB_REQUIRE(ctx != nullptr, "attn (static scratch): null context");
  HB_REQUIRE(B >= 1 && H >= 1 && Hkv >= 1 && H % Hkv == 0 && max_seq >= 1 && window >= 0 && D >= 1,
             "attn (static scratch): B=%d H=%d Hkv=%d D=%d max_seq=%d window=%d", B, H, Hkv, D,
             max_seq, window);
  // the split count the launch below will choose, hence the scratch it will touch
  const int eff_len = (window > 0 && window < max_seq) ? window : max_seq;
  const int nsplit = attn_pick_splits(ctx, B, Hkv, D, eff_len);
  const size_t need =
      nsplit > 1 ? (size_t)B * Hkv * nsplit * 8 * ((size_t)D + 2) * sizeof(float) : 0;
  if (need > (size_t)HB200_ATTN_STATIC_SCRATCH_BYTES) {
    set_error("attn (static scratch): this shape needs %zu bytes of split-K scratch but the "
              "built-in array holds %zu; call hb200_attn_decode with a workspace of your own",
              need, (size_t)HB200_ATTN_STATIC_SCRATCH_BYTES);
    return HB200_ERR_UNSUPPORTED;
  }
  int cur = -1;
  HB_CUDA(cudaGetDevice(&cur));
  HB_REQUIRE(cur == ctx->device,
             "attn (static scratch): device %d is current but the context belongs to device %d",
             cur, ctx->device);
  void*& addr = ctx->attn_static_addr;
  if (addr == nullptr) {  // first call of this context
    void* p = nullptr;
    HB_CUDA(cudaGetSymbolAddress(&p, g_attn_static_scratch));
    addr = p;
  }
  // Nothing in the array has to be cleared: every split writes its partial (max, sum, output
  // row) before the last split to arrive -- or the combine launch -- of the same call reads it.
  return hb200_attn_decode(ctx, d_q, q_is_f16, d_k, d_v, d_seqlens, B, H, Hkv, D, max_seq, window,
                           scale, addr, (size_t)HB200_ATTN_STATIC_SCRATCH_BYTES, d_out, stream);
}
