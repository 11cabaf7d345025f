// kquant_mma.cu -- batched (16..64 tokens per pass) Q4_K product with the dequantiser fused
// into the tensor-core kernel: the weights go from their 4.5-bit blocks to f16 in registers
// and from there straight into TENSOR MEMORY as the A operand of tcgen05.mma kind::f16; the
// f16 image of the tensor never exists in global memory.
//
// Same contract as the streaming Q4_K kernel (w = d*sc*q - dmin*m, f32 activations in, f32
// out; the reference's batched counterparts are the M>1 paths of Hesper/Layers/Linear.lean:
// 1152-1760,5973-6177).  Weights AND activations are rounded to f16 here (2^-11 each; the
// hi + lo activation split of the LM head would double the activation bytes every CTA pulls
// from L2, which is what bounds this kernel): measured error ~4e-4 of max|y|, bar 1e-3.
//
// One CTA per 128 weight rows, 11 warps with fixed roles:
//   warp 9     copies: one 2-D tensor-map TMA per super-block column of the tile (128 rows x
//              144 bytes, a 3-deep ring) and one 16 KB bulk copy of the step's activation
//              tiles (f16, operand layout written by the split kernel);
//   warps 0-7  dequantise: per step of 128 weights a thread owns one row and one 64-weight
//              chunk (two sub-blocks: 6-bit scale and min, 32 low and 32 high nibbles),
//              computes fma(d*sc, q, -dmin*m) in f32, packs f16 pairs and stores 32 columns
//              with one tcgen05.st;
//   warps 8,10 issue the 8 MMAs (M=128, N=64 tokens, K=16) of every other step into their
//              own f32 accumulator; tcgen05.commit releases the stage.
// Tensor memory: 2 x 64 accumulator columns + 6 stages x 64 columns of A.  Every wait is
// bounded; on expiry the kernel still releases its tensor memory.
#include <cuda_fp16.h>

#include "tcgen05.cuh"

namespace hb {

constexpr int kQmRows = 128;          // weight rows per CTA = MMA M
constexpr int kQmStepK = 128;         // weights per pipeline step (half a super-block)
constexpr int kQmACols = kQmStepK / 2;           // 64 TMEM columns of f16 pairs per stage
constexpr int kQmThreads = 352;

// What differs between the two formats: the bytes of 256 weights (one Q4_K super-block, eight
// Q8_0 blocks) and, with them, the box a copy brings and how deep the ring of boxes can be.
template <int FMT, int NT>
struct QmFmt {
  static constexpr int kUnit = FMT == 12 ? 144 : 272;
  static constexpr int kPkBytes = kQmRows * kUnit;  // 256 weights of every row: 18 / 34 KB
  static constexpr int kPkStages = (FMT == 12 || NT == 64) ? 3 : 2;
};

// NT tokens per pass = MMA N.  An MMA of this shape occupies the tensor pipe for the same
// ~128 cycles whether N is 64 or 256, so a pass over more tokens costs no extra tensor time;
// what grows is the accumulator (NT columns) and the activation tile every step brings.
template <int NT, int FMT = 12>
struct QmCfg {
  static constexpr int kIssuers = NT <= 128 ? 2 : 1;        // MMA-issuing warps, one accumulator each
  static constexpr int kA0 = kIssuers * NT;                 // first TMEM column of the A stages
  static constexpr int kStages = NT == 64 ? 6 : (NT == 128 ? 4 : 2);
  static constexpr int kBBytes = NT * kQmStepK * 2;         // activations per step: 16 / 32 / 64 KB
  static constexpr int kSmem =
      1024 + QmFmt<FMT, NT>::kPkStages * QmFmt<FMT, NT>::kPkBytes + kStages * kBBytes;
  static_assert(kA0 + kStages * kQmACols <= 512, "tensor memory columns");
  static_assert(kSmem <= 232448, "shared memory budget of one CTA");
};

constexpr int kQmMaxSeg = 3;  // tensors one launch multiplies by the same activations

struct QmSeg {
  const float* residual; // nullable; with glu != 0 it holds the gate values instead
  float* y;              // y[m * ldy + row]
  long ldy;
  int N;
  int tile0;             // first row tile of this tensor in the launch
  int glu;               // 0: y = acc (+ residual); 1: y = gelu_tanh(residual) * acc
};

struct QmParams {
  CUtensorMap tmap[kQmMaxSeg];  // blocks as [N rows][rowbytes], boxes of 128 rows x 144 bytes
  QmSeg seg[kQmMaxSeg];
  int nseg;
  const uint8_t* xb;     // f16 activations: [K/64][NT rows x 64 f16, operand layout]
  const float* rowscale; // [NT] power of two each token's row was divided by before rounding
  int K, M;
  int nsplit, bps;       // split-K: CTAs per row tile, super-block boxes per split
  float* part;           // [tile][split][NT tokens][128 rows] partial sums (nsplit > 1)
  int* tickets;          // [tile] arrival counters, zero between launches
  uint32_t idesc;
  uint32_t* status;
};


// 0.5*g*(1+tanh(sqrt(2/pi)*(g+0.044715 g^3))), the gate factor of the GeGLU
// (Hesper/Layers/FusedFFNSpec.lean:42-45), same expression as the standalone kernel
__device__ __forceinline__ float glu_gate(float g) {
  const float t = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.0f + tanhf(t));
}

__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// The four int8 of a word as f32 times d, packed to two f16 pairs.
__device__ __forceinline__ void q80_word(uint32_t w, float d, uint32_t& lo, uint32_t& hi) {
  const float a = d * (float)(int)(int8_t)(w & 0xFF), b = d * (float)(int)(int8_t)((w >> 8) & 0xFF);
  const float c = d * (float)(int)(int8_t)((w >> 16) & 0xFF), e = d * (float)(int)(int8_t)(w >> 24);
  lo = pack_f16(a, b);
  hi = pack_f16(c, e);
}

template <int NT, int FMT>
__global__ void __launch_bounds__(kQmThreads, 1) kq_mma_kernel(const __grid_constant__ QmParams p) {
  using Cfg = QmCfg<NT, FMT>;
  constexpr int kQmPkStages = QmFmt<FMT, NT>::kPkStages, kQmPkBytes = QmFmt<FMT, NT>::kPkBytes;
  constexpr int kUnit = QmFmt<FMT, NT>::kUnit;
  // a box dimension holds at most 256 elements: the 272-byte Q8_0 unit is mapped as 68 words
  constexpr int kBoxX = FMT == 12 ? 144 : 68;
  constexpr int kQmStages = Cfg::kStages, kQmBBytes = Cfg::kBBytes, kQmA0 = Cfg::kA0;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // this CTA's K range: whole super-blocks (boxes of 256 weights = 2 steps)
  const int tile = (int)blockIdx.x / p.nsplit, split = (int)blockIdx.x % p.nsplit;
  const int b0 = split * p.bps;
  const int nboxes = min(p.bps, p.K / 256 - b0);
  const int nsteps = 2 * nboxes;
  const int s0 = 2 * b0;  // first step, in units of the whole row
  int si = 0;
#pragma unroll
  for (int i = 1; i < kQmMaxSeg; ++i)
    if (i < p.nseg && tile >= p.seg[i].tile0) si = i;
  const QmSeg& sg = p.seg[si];
  const CUtensorMap* const tmap = &p.tmap[si];
  const int row0 = (tile - sg.tile0) * kQmRows;
  constexpr int kExpWarps = 8, kMmaWarpA = 8, kCopyWarp = 9, kMmaWarpB = 10;

  uint64_t* pk_full = reinterpret_cast<uint64_t*>(smem);  // [3] box landed (tx bytes)
  uint64_t* pk_free = pk_full + kQmPkStages;               // [3] every expander warp left it
  uint64_t* full = pk_free + kQmPkStages;   // [stages] A stored by 8 warps + activations landed
  uint64_t* mma_done = full + kQmStages;    // [stages] the MMAs that read the stage have retired
  uint64_t* done = mma_done + kQmStages;    // [1] both issuers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  uint8_t* pk = smem + 1024;
  uint8_t* bstg = pk + kQmPkStages * kQmPkBytes;

  if (tid == 0) {
    for (int i = 0; i < kQmPkStages; ++i) {
      mbar_init(&pk_full[i], 1);
      mbar_init(&pk_free[i], kExpWarps);
    }
    for (int i = 0; i < kQmStages; ++i) {
      mbar_init(&full[i], kExpWarps + 1);
      mbar_init(&mma_done[i], 1);
    }
    mbar_init(done, 2);
    fence_mbar_init();
  }
  if (warp == kMmaWarpA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(
        smem_u32(tmem_slot)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_before_sync();
  __syncthreads();
  tc_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (warp == kCopyWarp) {
    // ================= copies ==================================================================
    const uint64_t pol = policy_evict_first();
    auto issue_box = [&](int b) {
      if (lane == 0) {
        mbar_arrive_expect_tx(&pk_full[b % kQmPkStages], kQmPkBytes);
        tc_tma_box_2d(pk + (size_t)(b % kQmPkStages) * kQmPkBytes, tmap, (b0 + b) * kBoxX, row0,
                      &pk_full[b % kQmPkStages], pol);
      }
    };
    int bnext = 0;
    if (lane == 0)
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
    for (; bnext < kQmPkStages && bnext < nboxes; ++bnext) issue_box(bnext);  // weights: constant
    pdl_trigger();
    pdl_wait();  // the split activations come from the kernel before this one
    for (int s = 0; s < nsteps; ++s) {
      const int st = s % kQmStages;
      if (s >= kQmStages)
        ok = tc_wait(ok, &mma_done[st], (uint32_t)(((s / kQmStages) - 1) & 1), p.status);
      if (lane == 0) {
        mbar_arrive_expect_tx(&full[st], kQmBBytes);
        bulk_g2s(bstg + (size_t)st * kQmBBytes, p.xb + (size_t)(s0 + s) * kQmBBytes, kQmBBytes,
                 &full[st]);
      }
      if (bnext < nboxes && mbar_try_wait(&pk_free[bnext % kQmPkStages],
                                          (uint32_t)(((bnext / kQmPkStages) - 1) & 1))) {
        issue_box(bnext);
        ++bnext;
      }
    }
    while (bnext < nboxes) {
      ok = tc_wait(ok, &pk_free[bnext % kQmPkStages], (uint32_t)(((bnext / kQmPkStages) - 1) & 1),
                   p.status);
      if (!ok) break;
      issue_box(bnext);
      ++bnext;
    }
  } else if (warp == kMmaWarpA || warp == kMmaWarpB) {
    // ================= MMA issue: even steps -> accumulator 0, odd steps -> accumulator 1 =====
    const int which = warp == kMmaWarpA ? 0 : 1;
    const uint32_t tmem_d = tmem + (uint32_t)(which * NT);
    for (int s = which; s < nsteps && which < Cfg::kIssuers; s += Cfg::kIssuers) {
      const int st = s % kQmStages;
      ok = tc_wait(ok, &full[st], (uint32_t)((s / kQmStages) & 1), p.status);
      if (lane == 0) {
        tc_after_sync();
        const uint32_t a_t = tmem + kQmA0 + (uint32_t)st * kQmACols;
        const uint32_t bbase = smem_u32(bstg + (size_t)st * kQmBBytes);
#pragma unroll
        for (int j = 0; j < kQmStepK / 16; ++j)  // K = 16 per instruction: 8 columns of A
          tc_mma_f16_ta(tmem_d, a_t + j * 8,
                        tc_smem_desc(bbase + (j >> 2) * (kQmBBytes / 2) + (j & 3) * 256, 128, 1024, 0),
                        p.idesc, (s >= Cfg::kIssuers || j > 0) ? 1u : 0u);
        tc_commit(&mma_done[st]);
      }
      __syncwarp();
    }
    if (lane == 0) tc_commit(done);
  } else {
    // ================= dequantise into tensor memory ==========================================
    const int q = warp & 3, h = warp >> 2;       // lane quarter, which 64-weight chunk of the step
    const int erow = q * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16) + kQmA0 + 32u * h;
    for (int s = 0; s < nsteps; ++s) {
      const int st = s % kQmStages;
      const int box = s >> 1;
      const int c = ((s & 1) << 1) + h;          // chunk of the super-block: sub-blocks 2c, 2c+1
      if ((s & 1) == 0)
        ok = tc_wait(ok, &pk_full[box % kQmPkStages], (uint32_t)((box / kQmPkStages) & 1), p.status);
      if (s >= kQmStages) {
        ok = tc_wait(ok, &mma_done[st], (uint32_t)(((s / kQmStages) - 1) & 1), p.status);
        tc_after_sync();
      }
      uint32_t o[32];
      if (FMT == 12) {
        // super-block of this row: f16 d, f16 dmin, 12 bytes of 6-bit scales and mins, 128 bytes
        // of nibbles (Hesper/Quantization/Q4_K_M.lean:13-52,120-144)
        const uint8_t* blk = pk + (size_t)(box % kQmPkStages) * kQmPkBytes + (size_t)erow * 144;
        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
        const uint4 qa = *reinterpret_cast<const uint4*>(blk + 16 + 32 * c);
        const uint4 qb = *reinterpret_cast<const uint4*>(blk + 32 + 32 * c);
        const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
        // scale / min bytes j and j+1 (j = 2c) out of the 12 packed bytes hdr.y, hdr.z, hdr.w
        uint32_t sc2, m2;  // two 6-bit values each, in bytes 0 and 1
        if (c < 2) {
          sc2 = (hdr.y >> (16 * c)) & 0x3F3Fu;
          m2 = (hdr.z >> (16 * c)) & 0x3F3Fu;
        } else {
          const int sh = 16 * (c - 2);
          sc2 = ((hdr.w >> sh) & 0x0F0Fu) | (((hdr.y >> (sh + 6)) & 0x0303u) << 4);
          m2 = ((hdr.w >> (sh + 4)) & 0x0F0Fu) | (((hdr.z >> (sh + 6)) & 0x0303u) << 4);
        }
        const float ds0 = dd.x * (float)(sc2 & 0xFF), ds1 = dd.x * (float)(sc2 >> 8);
        const float dm0 = -(dd.y * (float)(m2 & 0xFF)), dm1 = -(dd.y * (float)(m2 >> 8));
        const uint32_t qq[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        // columns 0-15: sub-block 2c (low nibbles), 16-31: sub-block 2c+1 (high nibbles)
  #pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t w = qq[i];
          o[2 * i] = pack_f16(fmaf(ds0, (float)(w & 0xF), dm0), fmaf(ds0, (float)((w >> 8) & 0xF), dm0));
          o[2 * i + 1] = pack_f16(fmaf(ds0, (float)((w >> 16) & 0xF), dm0),
                                  fmaf(ds0, (float)((w >> 24) & 0xF), dm0));
          o[16 + 2 * i] = pack_f16(fmaf(ds1, (float)((w >> 4) & 0xF), dm1),
                                   fmaf(ds1, (float)((w >> 12) & 0xF), dm1));
          o[16 + 2 * i + 1] = pack_f16(fmaf(ds1, (float)((w >> 20) & 0xF), dm1),
                                       fmaf(ds1, (float)(w >> 28), dm1));
        }
      } else {
        // Q8_0 (Hesper/Layers/Linear.lean:6207-6223): blocks 2c and 2c+1 of the row's eight, 34
        // bytes each -- f16 d, then 32 int8.  The chunk starts on a word; block 2c's quants sit
        // two bytes into it (funnel shifts), block 2c+1's are word aligned.
        const uint32_t* wq = reinterpret_cast<const uint32_t*>(
            pk + (size_t)(box % kQmPkStages) * kQmPkBytes + (size_t)erow * kUnit + 68 * c);
        uint32_t w[17];
#pragma unroll
        for (int i = 0; i < 17; ++i) w[i] = wq[i];
        const float d0 = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
        const float d1 = __half2float(__ushort_as_half((unsigned short)(w[8] >> 16)));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          q80_word(__funnelshift_r(w[i], w[i + 1], 16), d0, o[2 * i], o[2 * i + 1]);
          q80_word(w[9 + i], d1, o[16 + 2 * i], o[16 + 2 * i + 1]);
        }
      }
      const uint32_t taddr = lane_addr + (uint32_t)st * kQmACols;
      HB_TMEM_ST32(taddr, o);
      if (s & 1) {  // second half of the super-block: this warp is done with the box
        __syncwarp();
        if (lane == 0)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(
                           smem_u32(&pk_free[box % kQmPkStages]))
                       : "memory");
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_before_sync();
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[st]))
                     : "memory");
    }
  }
  ok = tc_wait(true, done, 0, p.status) && ok;
  tc_after_sync();

  // ---- epilogue: lane = weight row, column = token; the issuers' accumulators add up.  Warp
  //      w owns lane quarter w & 3 and the 32-token groups w >> 2, (w >> 2) + 2, ... ----------
  const int q = warp & 3, r = q * 32 + lane;
  auto load_group = [&](int g, float (&acc)[32]) {  // tokens 32g .. 32g+31 of this row
    const uint32_t base = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(32 * g);
    uint32_t v[32];
    HB_TMEM_LD32(v, base);
    if (Cfg::kIssuers == 2) {
      uint32_t u[32];
      HB_TMEM_LD32(u, base + NT);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int t = 0; t < 32; ++t) acc[t] = __fadd_rn(__uint_as_float(v[t]), __uint_as_float(u[t]));
    } else {
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int t = 0; t < 32; ++t) acc[t] = __uint_as_float(v[t]);
    }
  };
  auto store_group = [&](int g, const float (&acc)[32]) {
    const int row = row0 + r, m0 = 32 * g;
    if (m0 >= p.M) return;  // the same for the whole warp
    const int mcount = min(32, p.M - m0);
    // lane t fetches token m0 + t's row scale, a shuffle hands it to every row
    const float my_rs = lane < mcount ? __ldcg(p.rowscale + m0 + lane) : 0.f;
    float res[32], rs[32];
#pragma unroll
    for (int t = 0; t < 32; ++t) rs[t] = __shfl_sync(0xffffffffu, my_rs, t);
    if (row >= sg.N || !ok) return;
    const size_t o0 = (size_t)m0 * sg.ldy + row;
    if (sg.residual) {
#pragma unroll
      for (int t = 0; t < 32; ++t) res[t] = t < mcount ? sg.residual[o0 + (size_t)t * sg.ldy] : 0.f;
    }
#pragma unroll
    for (int t = 0; t < 32; ++t)
      if (t < mcount) {
        float v = acc[t] * rs[t];
        if (sg.residual) v = sg.glu ? glu_gate(res[t]) * v : __fadd_rn(v, res[t]);
        sg.y[o0 + (size_t)t * sg.ldy] = v;
      }
  };
  if (p.nsplit == 1) {
    if (warp < kExpWarps)
      for (int g = warp >> 2; g < NT / 32; g += 2) {
        float acc[32];
        load_group(g, acc);
        store_group(g, acc);
      }
  } else {
    // split-K: every split publishes its partial; the last one to arrive (a ticket per row
    // tile) adds ALL partials in split order, so the f32 result does not depend on who it was
    __shared__ int s_last;
    float* mine = p.part + ((size_t)(tile * p.nsplit + split) * NT) * kQmRows;
    if (warp < kExpWarps)
      for (int g = warp >> 2; g < NT / 32; g += 2) {
        if (32 * g >= p.M) continue;
        float acc[32];
        load_group(g, acc);
#pragma unroll
        for (int t = 0; t < 32; ++t) mine[(size_t)(32 * g + t) * kQmRows + r] = acc[t];
      }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int t = atomicAdd(&p.tickets[tile], 1);
      s_last = (t == p.nsplit - 1);
      if (s_last) p.tickets[tile] = 0;
    }
    __syncthreads();
    if (s_last && warp < kExpWarps) {
      __threadfence();
      for (int g = warp >> 2; g < NT / 32; g += 2) {
        if (32 * g >= p.M) continue;
        float acc[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) acc[t] = 0.f;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
          const float* other =
              p.part + ((size_t)(tile * p.nsplit + s2) * NT + 32 * g) * kQmRows + r;
#pragma unroll
          for (int t = 0; t < 32; ++t) acc[t] = __fadd_rn(acc[t], __ldcg(other + (size_t)t * kQmRows));
        }
        store_group(g, acc);
      }
    }
  }
  tc_before_sync();
  __syncthreads();
  if (warp == kMmaWarpA)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem));
}

}  // namespace hb

using namespace hb;

template <int NT, int FMT>
static int kq_mma_launch(hb200_ctx* ctx, QmParams& p, int tiles, cudaStream_t st) {
  using Cfg = QmCfg<NT, FMT>;
  // kind::f16: D = f32, A and B f16, both K-major, N = NT, M = 128
  p.idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kQmRows >> 4) << 24);
  // split-K: the launch takes ceil(tiles * s / SMs) waves of CTAs that each do 1/s of a row
  // tile's work plus a fixed part (pipeline fill, tensor-memory allocation, the partials'
  // round trip: taken as a tenth of a tile).  Pick the s that minimises waves * (1/s + 0.1):
  // few row tiles spread over the idle SMs (20 tiles -> 7 splits), and a tile count just above
  // a multiple of the SM count no longer costs a whole extra wave (160 tiles: 2 waves of full
  // tiles -> 4 waves of thirds).  Each split at least 2 super-blocks long, partials within
  // their scratch region, tickets within theirs.
  const int nboxes = p.K / 256;
  int nsplit = 1;
  {
    float best = 1e30f;
    for (int s2 = 1; s2 <= nboxes / 2 || s2 == 1; ++s2) {
      if (s2 > 1 && (size_t)tiles * s2 * NT * kQmRows * 4 > kScratchBytes - kScratchSplitK) break;
      const int waves = (tiles * s2 + ctx->sm_count - 1) / ctx->sm_count;
      const float cost = (float)waves * (1.0f / (float)s2 + 0.1f);
      if (cost < best - 1e-6f) {
        best = cost;
        nsplit = s2;
      }
    }
  }
  if (nsplit < 1 || tiles > kCtxTickets) nsplit = 1;
  p.bps = (nboxes + nsplit - 1) / nsplit;
  p.nsplit = (nboxes + p.bps - 1) / p.bps;  // no empty split
  {
    const int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(kq_mma_kernel<NT, FMT>), (size_t)Cfg::kSmem);
    if (rc != HB200_OK) return rc;
  }
  HB_CUDA(launch_pdl(kq_mma_kernel<NT, FMT>, dim3((unsigned)(tiles * p.nsplit)), dim3(kQmThreads),
                     (size_t)Cfg::kSmem, st, ctx->pdl, p));
  return HB200_OK;
}

// For each of nseg tensors: y[m*ldy + n] = sum_k dequant(W)[n,k] x[m,k] (+ residual) for the
// M <= NT tokens staged by hb_gemm16_split (dtype f16, single term, NT token rows per block;
// NT = 64, 128 or 256), all in ONE launch.  glu != 0: `residual` holds gate pre-activations
// and y = gelu_tanh(gate) * product (y may be the same array as residual; the gate values
// must come from an earlier launch).  Q4_K or Q8_0 (fmt: the GGUF type id); K a multiple of 256.
int hb_kq_mma_run_multi(hb200_ctx* ctx, const HbKqSeg* segs, int nseg, int K, int M, int NT,
                        cudaStream_t st, int fmt) {
  HB_REQUIRE(fmt == HB200_FMT_Q4_K || fmt == HB200_FMT_Q8_0, "kquant (fused batched): format %d", fmt);
  HB_REQUIRE(nseg >= 1 && nseg <= kQmMaxSeg && K % 256 == 0 && M >= 1 && M <= NT &&
                 (NT == 64 || NT == 128 || NT == 256),
             "kquant (fused batched): nseg=%d K=%d M=%d NT=%d", nseg, K, M, NT);
  QmParams p = {};
  TcEncodeTiledFn encode = tc_tensor_map_encoder();
  HB_REQUIRE(encode != nullptr, "kquant (fused batched): the driver has no cuTensorMapEncodeTiled");
  const int unit = fmt == HB200_FMT_Q4_K ? 144 : 272;  // bytes of 256 weights
  const int rowbytes = K / 256 * unit;
  int tiles = 0;
  for (int s = 0; s < nseg; ++s) {
    const HbKqSeg& g = segs[s];
    HB_REQUIRE(g.N >= 1 && g.N < (1l << 31) && g.blocks && g.y,
               "kquant (fused batched): tensor %d has no rows or a null pointer", s);
    HB_REQUIRE(!g.glu || g.residual, "kquant (fused batched): GLU epilogue without gate values");
    // Q4_K: bytes; Q8_0: 32-bit words (a box dimension holds at most 256 elements, 272 > 256)
    const int esz = fmt == HB200_FMT_Q4_K ? 1 : 4;
    const cuuint64_t dims[2] = {(cuuint64_t)(rowbytes / esz), (cuuint64_t)g.N};
    const cuuint64_t strides[1] = {(cuuint64_t)rowbytes};
    const cuuint32_t box[2] = {(cuuint32_t)(unit / esz), (cuuint32_t)kQmRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = encode(&p.tmap[s],
                               esz == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2,
                               const_cast<uint8_t*>(g.blocks), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HB_REQUIRE(rc == CUDA_SUCCESS, "kquant (fused batched): cuTensorMapEncodeTiled failed (%d)",
               (int)rc);
    p.seg[s] = {g.residual, g.y, g.ldy, (int)g.N, tiles, g.glu};
    tiles += (int)((g.N + kQmRows - 1) / kQmRows);
  }
  p.nseg = nseg;
  p.xb = static_cast<const uint8_t*>(ctx->d_scratch) + kScratchLmSplit;
  p.rowscale = reinterpret_cast<const float*>(static_cast<const uint8_t*>(ctx->d_scratch) +
                                              kScratchRowScale);
  p.K = K;
  p.M = M;
  p.part = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->d_scratch) + kScratchSplitK);
  p.tickets = ctx->d_tickets;
  p.status = ctx->d_status;
  if (fmt == HB200_FMT_Q4_K) {
    switch (NT) {
      case 64: return kq_mma_launch<64, 12>(ctx, p, tiles, st);
      case 128: return kq_mma_launch<128, 12>(ctx, p, tiles, st);
      default: return kq_mma_launch<256, 12>(ctx, p, tiles, st);
    }
  }
  switch (NT) {
    case 64: return kq_mma_launch<64, 8>(ctx, p, tiles, st);
    case 128: return kq_mma_launch<128, 8>(ctx, p, tiles, st);
    default: return kq_mma_launch<256, 8>(ctx, p, tiles, st);
  }
}

int hb_kq_mma_run(hb200_ctx* ctx, const uint8_t* d_blocks, int K, long N, int M, int NT,
                  float* d_y, const float* d_residual, long ldy, int glu, cudaStream_t st, int fmt) {
  const HbKqSeg g = {d_blocks, N, d_y, d_residual, ldy, glu};
  return hb_kq_mma_run_multi(ctx, &g, 1, K, M, NT, st, fmt);
}
