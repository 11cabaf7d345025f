// bitlinear_mma.cu -- batched (16..64 tokens) ternary i2_s x int8 product on the 5th-generation
// tensor cores: tcgen05.mma kind::i8 with the int32 accumulator in tensor memory.
//
// Same arithmetic contract as the batch-1 kernel (bit-exact int32 accumulators, then
// y = ((float)acc*d)*s (+residual)); the reference's counterparts are the tiled and WMMA
// M>1 paths of BitLinear (Hesper/Layers/BitLinear.lean:122,869,994).  With 16 or more
// tokens per weight the op is a real contraction, so the weights are still streamed once
// but the multiply-accumulates move from dp4a to the tensor core:
//
//   quant_act_kernel   one CTA per token: optional RMSNorm, absmax int8 quantisation; the
//                      int8 activations are written straight in the shared-memory operand
//                      layout (K-major, 8x16-byte core matrices), one 8 KB block per
//                      128-wide K group, so the GEMM kernel fetches a B tile with ONE bulk copy
//   bitlinear_mma_kernel  one CTA per 128 weight rows, 11 warps with fixed roles:
//     * warp 9 issues every copy: the packed weights as boxes of 128 rows x 128 bytes
//       (4 groups) through a 2-D tensor map with the 128-byte swizzle, ONE instruction per
//       16 KB on a 4-deep ring (per-row 1-D bulk copies cost ~35 ns each at the TMA unit and
//       throttled the stream), and each step's activations with one 16 KB bulk copy;
//     * warps 0-7 expand two 128-wide groups per step from 2-bit codes to unsigned bytes
//       (0,1,2) and store them with tcgen05.st straight into TENSOR MEMORY as the A operand
//       (lane = weight row, 4 K-bytes per column): the expanded weights never touch shared
//       memory, whose bandwidth bounded the earlier shared-memory-A version of this kernel;
//     * warps 8 and 10 each issue the MMAs of every other step from one thread into their own
//       accumulator (tcgen05.mma kind::i8, A from tensor memory, B by a shared-memory
//       descriptor, M=128, N=64 tokens, K=32 per instruction; 2 x 64 columns of int32): one
//       thread alone spends ~45 ns per MMA, two keep the tensor pipe busy.  One barrier per
//       step gathers the 8 expander arrivals and the activation bytes; one tcgen05.commit
//       per step releases the stage (6 stages = 384 columns of A);
//     * epilogue: 8 warps read 32 lanes x 32 columns of both accumulators (tcgen05.ld
//       32x32b), add them, subtract sum(q) per token (value = code - 1), scale and store;
//     * split-K: a launch with few tiles (o_proj and down_proj have 20) splits K over several
//       CTAs per tile; each publishes its int32 partial, the last to arrive (a ticket per
//       tile) adds the others' and runs the epilogue -- exact, since integers commute.
// Every mbarrier wait is bounded; on expiry the kernel still releases its tensor memory.
#include "tcgen05.cuh"

namespace hb {

constexpr int kMmaThreads = 256;
constexpr int kMmaRows = 128;    // weight rows per CTA = MMA M
constexpr int kMmaTokens = 64;   // MMA N of the narrow variant (16..64 tokens)
constexpr int kChunkGroups = 4;  // 128-weight groups per packed box: 128 bytes of every row
constexpr int kPkStages = 4;     // packed ring
constexpr int kPkBytes = kMmaRows * kChunkGroups * 32;  // 16 KB box
constexpr int kStepGroups = 2;   // groups per pipeline step: one barrier round trip per 8 MMAs
constexpr int kAGroupCols = 32;  // TMEM columns of one expanded group: 128 K-bytes per row
constexpr int kMmaCtrl = 2048;   // barriers, tensor-memory slot, d[NT], sum(q)[NT]

// NT tokens per pass = MMA N: 64, or 128 for the prompt passes (half the weight passes per
// token).  Tensor memory, 512 columns: accumulator of the first issuing warp at 0, the A stages
// behind it, the second warp's accumulator in the last NT columns.
template <int NT>
struct MmaCfg {
  static constexpr int kStages = NT == 64 ? 6 : 4;  // operand stages (A in TMEM, B in smem)
  static constexpr int kBBytes = NT * 128;          // activation tile of one 128-wide group
  static constexpr int kA0 = NT;                    // first column of the A stages
  static constexpr int kAcc1 = 512 - NT;            // the second accumulator
  static constexpr int kSmem = kMmaCtrl + kPkStages * kPkBytes + kStages * kStepGroups * kBBytes;
  // kind::i8: D = s32, A = u8, B = s8, both K-major, N = NT, M = 128
  static constexpr uint32_t kIdesc = (2u << 4) | (0u << 7) | (1u << 10) |
                                     ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kMmaRows >> 4) << 24);
  static_assert(kA0 + kStages * kStepGroups * kAGroupCols <= kAcc1, "tensor memory columns");
  static_assert(kSmem <= 232448, "shared memory budget of one CTA");
};

struct MmaSeg {
  const uint8_t* w;
  const float* scale;
  const float* residual;
  float* y;
  int32_t* acc;
  int N;
  int tile0;
};

struct MmaParams {
  CUtensorMap tmap[4];  // per segment: packed weights as [N rows][K/4 bytes], 128 x 128 boxes
  MmaSeg seg[4];
  int nseg, K, M;
  int nsplit, gps;     // split-K: CTAs per tile, groups per split
  int32_t* part;       // [tile][split][NT tokens][128 rows] partial accumulators (nsplit > 1)
  int* tickets;        // [tile] arrival counters, zero between launches
  const uint8_t* xq;   // [K/128][NT tokens x 128 bytes, core-matrix layout]
  const float* d;      // [NT] activation scales
  const int32_t* sumq; // [NT]
  uint32_t* status;
};

// ---- activation quantiser -------------------------------------------------------------

struct QuantParams {
  const float* x;      // [M][K]
  const float* gamma;  // nullable
  float eps;
  int K, M;
  uint8_t* xq;
  float* d;
  int32_t* sumq;
  float* act_scale;    // nullable user copy of d
  int bbytes;          // bytes of one 128-wide K group of the tile: tokens per pass x 128
};

__global__ void __launch_bounds__(256) quant_act_kernel(const __grid_constant__ QuantParams p) {
  __shared__ double red_d[8];
  __shared__ uint32_t red_u[8];
  __shared__ int red_i[8];
  extern __shared__ __align__(16) float xs[];  // [K]
  pdl_trigger();
  if (p.gamma)  // constants of the model: into L1 before the wait on the previous kernel
    for (int i = threadIdx.x * 32; i < p.K; i += 256 * 32)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gamma + i));
  pdl_wait();
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, nvec = K >> 2;
  auto dst_of = [&](int i) {  // float4 index -> byte offset of its 4 int8 in the operand layout
    const int k = i << 2;
    return (size_t)(k >> 7) * p.bbytes + (size_t)(m >> 3) * 1024 + (size_t)((k & 127) >> 4) * 128 +
           (size_t)(m & 7) * 16 + (k & 15);
  };
  if (m >= p.M) {  // padding token of the tile
    for (int i = tid; i < nvec; i += 256) *reinterpret_cast<uint32_t*>(p.xq + dst_of(i)) = 0u;
    if (tid == 0) {
      p.d[m] = 0.f;
      p.sumq[m] = 0;
    }
    return;
  }
  const float4* xg = reinterpret_cast<const float4*>(p.x + (size_t)m * K);
  float4* x4 = reinterpret_cast<float4*>(xs);
  float amax = 0.f;
  if (p.gamma) {
    double ss = 0.0;
    for (int i = tid; i < nvec; i += 256) {
      const float4 v = __ldcg(xg + i);
      x4[i] = v;
      ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) red_d[warp] = ss;
    __syncthreads();
    ss = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += red_d[i];
    const float rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
    const float4* gg = reinterpret_cast<const float4*>(p.gamma);
    for (int i = tid; i < nvec; i += 256) {
      float4 v = x4[i];
      const float4 g = __ldg(gg + i);
      v.x = __fmul_rn(__fmul_rn(v.x, rinv), g.x);
      v.y = __fmul_rn(__fmul_rn(v.y, rinv), g.y);
      v.z = __fmul_rn(__fmul_rn(v.z, rinv), g.z);
      v.w = __fmul_rn(__fmul_rn(v.w, rinv), g.w);
      x4[i] = v;
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
  } else {
    for (int i = tid; i < nvec; i += 256) {
      const float4 v = __ldcg(xg + i);
      x4[i] = v;
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
  }
  const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
  if (lane == 0) red_u[warp] = wmax;
  __syncthreads();
  uint32_t mx = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) mx = max(mx, red_u[i]);
  amax = __uint_as_float(mx);
  const float d = __fdiv_rn(amax, 127.0f);
  const float inv = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
  int sumq = 0;
  for (int i = tid; i < nvec; i += 256) {
    const float4 v = x4[i];
    const int q0 = __float2int_rn(__fmul_rn(v.x, inv)), q1 = __float2int_rn(__fmul_rn(v.y, inv));
    const int q2 = __float2int_rn(__fmul_rn(v.z, inv)), q3 = __float2int_rn(__fmul_rn(v.w, inv));
    sumq += (q0 + q1) + (q2 + q3);
    *reinterpret_cast<uint32_t*>(p.xq + dst_of(i)) =
        (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) | ((uint32_t)(q2 & 0xff) << 16) |
        ((uint32_t)q3 << 24);
  }
  sumq = __reduce_add_sync(0xffffffffu, sumq);
  if (lane == 0) red_i[warp] = sumq;
  __syncthreads();
  if (tid == 0) {
    int s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red_i[i];
    p.d[m] = d;
    p.sumq[m] = s;
    if (p.act_scale) p.act_scale[m] = d;
  }
}

// ---- tcgen05 helpers --------------------------------------------------------------------

// A operand from tensor memory (lane = weight row, 4 K-bytes per 32-bit column).
__device__ __forceinline__ void umma_i8_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int NT>
__global__ void __launch_bounds__(kMmaThreads + 96, 1)
    bitlinear_mma_kernel(const __grid_constant__ MmaParams p) {
  using Cfg = MmaCfg<NT>;
  constexpr int kStages = Cfg::kStages, kBBytes = Cfg::kBBytes;
  constexpr int NCH = NT / 64;  // 32-token chunks an epilogue warp owns
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // this CTA's K range (split-K over 128-wide groups; a whole row when nsplit == 1)
  const int tile = (int)blockIdx.x / p.nsplit, split = (int)blockIdx.x % p.nsplit;
  const int gbase = split * p.gps;
  const int ngroups = min(p.gps, (p.K >> 7) - gbase);
  const int nchunks = (ngroups + kChunkGroups - 1) / kChunkGroups;
  const int nsteps = (ngroups + kStepGroups - 1) / kStepGroups;
  constexpr int kExpWarps = kMmaThreads / 32;  // warps 0..7 expand, warp 8 issues MMAs, warp 9 copies
  constexpr int kMmaWarp = kExpWarps, kCopyWarp = kExpWarps + 1;

  // control block, then the packed ring and the activation stages (1 KB aligned)
  uint64_t* pk_full = reinterpret_cast<uint64_t*>(smem);  // [kPkStages] box landed (tx bytes)
  uint64_t* pk_free = pk_full + kPkStages;                 // [kPkStages] every expander warp left it
  uint64_t* full = pk_free + kPkStages;   // [kStages] A stored by 8 warps + B landed (tx bytes)
  uint64_t* mma_done = full + kStages;    // [kStages] the MMAs that read the stage have retired
  uint64_t* done = mma_done + kStages;    // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  float* sd = reinterpret_cast<float*>(smem + 512);        // [NT]
  int* ssum = reinterpret_cast<int*>(smem + 1024);         // [NT]
  uint8_t* pk = smem + kMmaCtrl;
  uint8_t* bstg = pk + kPkStages * kPkBytes;  // [kStages][kStepGroups] activation tiles

  // tile -> (segment, first row)
  int seg = 0;
#pragma unroll
  for (int s = 1; s < 4; ++s)
    if (s < p.nseg && tile >= p.seg[s].tile0) seg = s;
  const int seg_N = p.seg[seg].N;
  const int row0 = (tile - p.seg[seg].tile0) * kMmaRows;
  const int nrows = min(kMmaRows, seg_N - row0);

  if (tid == 0) {
    for (int i = 0; i < kPkStages; ++i) {
      mbar_init(&pk_full[i], 1);
      mbar_init(&pk_free[i], kExpWarps);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], kExpWarps + 1);
      mbar_init(&mma_done[i], 1);
    }
    mbar_init(done, 2);
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {  // all 512 columns: two accumulators, the A stages between them
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
    // ================= copy warp: packed weight boxes and activation tiles ==================
    const uint64_t pol = policy_evict_first();
    const CUtensorMap* tm = &p.tmap[seg];
    int cnext = 0;
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tm)) : "memory");
      for (; cnext < kPkStages && cnext < nchunks; ++cnext) {  // weights: no dependency
        mbar_arrive_expect_tx(&pk_full[cnext], kPkBytes);
        tc_tma_box_2d(pk + (size_t)cnext * kPkBytes, tm, (gbase + cnext * kChunkGroups) * 32, row0,
                   &pk_full[cnext], pol);
      }
    }
    cnext = min(kPkStages, nchunks);
    pdl_trigger();
    pdl_wait();  // the quantised activations come from the kernel before this one
    for (int s = 0; s < nsteps; ++s) {
      const int st = s % kStages;
      if (s >= kStages)  // the MMAs that read this stage kStages steps ago must have retired
        ok = tc_wait(ok, &mma_done[st], (uint32_t)(((s / kStages) - 1) & 1), p.status);
      if (lane == 0) {  // activations of the step's groups: contiguous in the operand layout
        const int g0 = s * kStepGroups;
        const uint32_t bytes = (uint32_t)min(kStepGroups, ngroups - g0) * kBBytes;
        mbar_arrive_expect_tx(&full[st], bytes);
        bulk_g2s(bstg + (size_t)st * kStepGroups * kBBytes, p.xq + (size_t)(gbase + g0) * kBBytes, bytes,
                 &full[st]);
      }
      // refill the packed ring as soon as every expander warp has left the oldest box
      if (cnext < nchunks && mbar_try_wait(&pk_free[cnext % kPkStages],
                                           (uint32_t)(((cnext / kPkStages) - 1) & 1))) {
        if (lane == 0) {
          mbar_arrive_expect_tx(&pk_full[cnext % kPkStages], kPkBytes);
          tc_tma_box_2d(pk + (size_t)(cnext % kPkStages) * kPkBytes, tm,
                     (gbase + cnext * kChunkGroups) * 32, row0, &pk_full[cnext % kPkStages], pol);
        }
        ++cnext;
      }
    }
    while (cnext < nchunks) {  // boxes still owed (their slot frees up as the expanders go)
      ok = tc_wait(ok, &pk_free[cnext % kPkStages], (uint32_t)(((cnext / kPkStages) - 1) & 1),
                    p.status);
      if (!ok) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(&pk_full[cnext % kPkStages], kPkBytes);
        tc_tma_box_2d(pk + (size_t)(cnext % kPkStages) * kPkBytes, tm,
                   (gbase + cnext * kChunkGroups) * 32, row0, &pk_full[cnext % kPkStages], pol);
      }
      ++cnext;
    }
  } else if (warp == kMmaWarp || warp == kMmaWarp + 2) {
    // ================= two MMA warps: even steps -> accumulator 0, odd steps -> accumulator 1
    const int which = warp == kMmaWarp ? 0 : 1;
    const uint32_t tmem_d = tmem + (which ? (uint32_t)Cfg::kAcc1 : 0u);
    for (int s = which; s < nsteps; s += 2) {
      const int st = s % kStages;
      ok = tc_wait(ok, &full[st], (uint32_t)((s / kStages) & 1), p.status);
      if (lane == 0) {
        tc_after_sync();
        const uint32_t a_t = tmem + Cfg::kA0 + (uint32_t)st * (kStepGroups * kAGroupCols);
        const uint32_t bbase = smem_u32(bstg + (size_t)st * kStepGroups * kBBytes);
        const int ng = min(kStepGroups, ngroups - s * kStepGroups);
#pragma unroll
        for (int gg = 0; gg < kStepGroups; ++gg)
          if (gg < ng) {
#pragma unroll
            for (int j = 0; j < 4; ++j)  // K = 32 bytes per instruction: 8 columns of A
              umma_i8_ta(tmem_d, a_t + gg * kAGroupCols + j * 8,
                         tc_smem_desc(bbase + gg * kBBytes + j * 256, 128, 1024, 0), Cfg::kIdesc,
                         (s > 1 || gg > 0 || j > 0) ? 1u : 0u);
          }
        tc_commit(&mma_done[st]);  // arrives once these (and all earlier) MMAs have retired
      }
      __syncwarp();
    }
    if (lane == 0) tc_commit(done);
  } else {
    // ================= expander warps ========================================================
    // warp w owns TMEM lanes (= weight rows) 32*(w&3).., and K-half h = w>>2 of every group:
    // planes 2h and 2h+1 of the packed bytes = K bytes 64h..64h+63 = 16 columns.
    const int q = warp & 3, h = warp >> 2;
    const int erow = q * 32 + lane;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16) + Cfg::kA0 + 16u * h;
    for (int s = 0; s < nsteps; ++s) {
      const int st = s % kStages;
      if (s >= kStages) {
        ok = tc_wait(ok, &mma_done[st], (uint32_t)(((s / kStages) - 1) & 1), p.status);
        tc_after_sync();
      }
      const int ng = min(kStepGroups, ngroups - s * kStepGroups);
#pragma unroll
      for (int gg = 0; gg < kStepGroups; ++gg) {
        if (gg >= ng) break;
        const int g = s * kStepGroups + gg;
        const int c = g / kChunkGroups, gi = g % kChunkGroups;
        if (gi == 0)
          ok = tc_wait(ok, &pk_full[c % kPkStages], (uint32_t)((c / kPkStages) & 1), p.status);
        // the row's 32 packed bytes of this group: units 2gi and 2gi+1 of its swizzled 128 bytes
        const uint8_t* rowp = pk + (size_t)(c % kPkStages) * kPkBytes + (size_t)erow * 128;
        const uint4 w0 = *reinterpret_cast<const uint4*>(rowp + (((2 * gi) ^ (erow & 7)) << 4));
        const uint4 w1 = *reinterpret_cast<const uint4*>(rowp + (((2 * gi + 1) ^ (erow & 7)) << 4));
        const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        uint32_t o[16];
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
          // plane pl holds elements 32*pl + j in byte j: word i -> K bytes 32*pl + 4i .. +3
          const int sh = h ? (2 - 2 * pp) : (6 - 2 * pp);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[8 * pp + i] = (w[i] >> sh) & 0x03030303u;
        }
        const uint32_t taddr = lane_addr + (uint32_t)st * (kStepGroups * kAGroupCols) +
                               (uint32_t)gg * kAGroupCols;
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
            "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]),
            "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]), "r"(o[14]),
            "r"(o[15])
            : "memory");
        if (gi == kChunkGroups - 1 || g == ngroups - 1) {  // last read of this packed box
          __syncwarp();
          if (lane == 0)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(
                             smem_u32(&pk_free[c % kPkStages]))
                         : "memory");
        }
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      tc_before_sync();
      __syncwarp();
      if (lane == 0)
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&full[st]))
                     : "memory");
    }
    pdl_wait();  // d and sum(q) come from the quantiser
    if (tid < NT) {
      sd[tid] = p.d[tid];
      ssum[tid] = p.sumq[tid];
    }
  }
  ok = tc_wait(true, done, 0, p.status) && ok;
  tc_after_sync();
  __syncthreads();  // sd / ssum visible; every warp past its loop

  // ---- epilogue: TMEM lane = weight row, column = token.  Warps w and w + 4 share a lane
  //      quarter; a warp owns the 32-token chunks (w >> 2), (w >> 2) + 2, ... ----------------
  const int q = warp & 3, half = warp >> 2;  // lane quarter, first chunk (expander warps only)
  const int r = q * 32 + lane;
  uint32_t v[NCH][32];
  if (warp < kExpWarps) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)((half + 2 * c) * 32);
      HB_TMEM_LD32(v[c], taddr);
      if (nsteps > 1) {  // the second MMA warp's accumulator
        uint32_t u[32];
        HB_TMEM_LD32(u, taddr + (uint32_t)Cfg::kAcc1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int t = 0; t < 32; ++t) v[c][t] += u[t];
      } else {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
    }
  }

  // ---- split-K: publish the int32 partial, the last split of the tile to arrive adds them ---
  // Integer addition commutes, so the result is bit-identical to the unsplit product.
  bool finish = true;
  if (p.nsplit > 1) {
    __shared__ int s_last;
    int32_t* mine = p.part + ((size_t)(tile * p.nsplit + split) * NT) * kMmaRows;
    if (warp < kExpWarps) {
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int m0 = (half + 2 * c) * 32;
        if (m0 >= p.M) continue;
#pragma unroll
        for (int t = 0; t < 32; ++t) mine[(size_t)(m0 + t) * kMmaRows + r] = (int32_t)v[c][t];
      }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int t = atomicAdd(&p.tickets[tile], 1);
      s_last = (t == p.nsplit - 1);
      if (s_last) p.tickets[tile] = 0;  // every split has arrived: ready for the next launch
    }
    __syncthreads();
    finish = s_last != 0;
    if (finish && warp < kExpWarps) {
      __threadfence();
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int m0 = (half + 2 * c) * 32;
        if (m0 >= p.M) continue;
        for (int s2 = 0; s2 < p.nsplit; ++s2) {
          if (s2 == split) continue;
          const int32_t* other = p.part + ((size_t)(tile * p.nsplit + s2) * NT + m0) * kMmaRows + r;
#pragma unroll
          for (int t = 0; t < 32; ++t) v[c][t] += (uint32_t)__ldcg(other + (size_t)t * kMmaRows);
        }
      }
    }
  }

  if (finish && warp < kExpWarps) {
    const float ws = __ldg(p.seg[seg].scale);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int m0 = (half + 2 * c) * 32;
      if (r < nrows && ok && m0 < p.M) {
        const int mcount = min(32, p.M - m0);
        const size_t o0 = (size_t)m0 * seg_N + row0 + r;
        float* yp = p.seg[seg].y + o0;
        const float* rp = p.seg[seg].residual ? p.seg[seg].residual + o0 : nullptr;
        int32_t* ap = p.seg[seg].acc ? p.seg[seg].acc + o0 : nullptr;
        // all shared-memory reads first (v[t] becomes the integer total), so that the stores
        // below, whose target the compiler cannot tell from shared memory, do not serialise them
        float dsc[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          v[c][t] = (uint32_t)((int)v[c][t] - ssum[m0 + t]);
          dsc[t] = sd[m0 + t];
        }
        if (ap) {
#pragma unroll
          for (int t = 0; t < 32; ++t)
            if (t < mcount) ap[(size_t)t * seg_N] = (int)v[c][t];
        }
        float res[32];
        if (rp) {
#pragma unroll
          for (int t = 0; t < 32; ++t) res[t] = t < mcount ? rp[(size_t)t * seg_N] : 0.f;
        }
#pragma unroll
        for (int t = 0; t < 32; ++t)
          if (t < mcount) {
            float y = __fmul_rn(__fmul_rn((float)(int)v[c][t], dsc[t]), ws);
            if (rp) y = __fadd_rn(y, res[t]);
            yp[(size_t)t * seg_N] = y;
          }
      }
    }
  }
  tc_before_sync();
  __syncthreads();
  if (warp == kMmaWarp)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem));
}

}  // namespace hb

using namespace hb;

// Batched path of hb200_bitlinear_forward_multi (16 <= M <= 128: one pass of 64 or 128 token
// slots).  Scratch in the context: quantised activations in operand layout, their scales and
// sums.
template <int NT>
static int bl_mma_launch(hb200_ctx* ctx, MmaParams& p, int tiles, cudaStream_t st) {
  // split-K when the tiles alone leave most SMs idle: as many splits as fit the SMs, each at
  // least 4 groups (two pipeline steps) long, partials within their scratch region
  const int ngroups = p.K / 128;
  int nsplit = ctx->sm_count / tiles;
  if (nsplit > ngroups / 4) nsplit = ngroups / 4;
  while (nsplit > 1 &&
         (size_t)tiles * nsplit * NT * kMmaRows * 4 > kScratchBytes - kScratchSplitK)
    --nsplit;
  if (nsplit < 1 || tiles > kCtxTickets) nsplit = 1;
  p.gps = (ngroups + nsplit - 1) / nsplit;
  p.nsplit = (ngroups + p.gps - 1) / p.gps;  // no empty split
  const int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(bitlinear_mma_kernel<NT>),
                              (size_t)MmaCfg<NT>::kSmem);
  if (rc != HB200_OK) return rc;
  HB_CUDA(launch_pdl(bitlinear_mma_kernel<NT>, dim3(tiles * p.nsplit), dim3(kMmaThreads + 96),
                     (size_t)MmaCfg<NT>::kSmem, st, ctx->pdl, p));
  return HB200_OK;
}

int hb_bitlinear_mma_run(hb200_ctx* ctx, const hb200_bitlinear_seg* segs, int nseg, int K,
                         const float* d_x, int M, const float* d_rms_gamma, float rms_eps,
                         float* d_act_scale, cudaStream_t st) {
  ScratchUse use(ctx, st);  // quantised activation tiles, split-K partials, tickets
  HB_REQUIRE(M >= 1 && M <= 128, "bitlinear (batched): %d tokens in one pass (at most 128)", M);
  const int NT = M <= 64 ? 64 : 128;
  const size_t xq_bytes = (size_t)(K / 128) * NT * 128;
  HB_REQUIRE(xq_bytes + 1024 <= kScratchGlu,
             "bitlinear (batched): K=%d needs %zu bytes of activation scratch", K, xq_bytes);
  uint8_t* base = static_cast<uint8_t*>(ctx->d_scratch);
  float* d = reinterpret_cast<float*>(base);            // [128]
  int32_t* sumq = reinterpret_cast<int32_t*>(base + 512);  // [128]
  uint8_t* xq = base + 1024;
  QuantParams q = {d_x, d_rms_gamma, rms_eps, K, M, xq, d, sumq, d_act_scale, NT * 128};
  HB_CUDA(launch_pdl(quant_act_kernel, dim3(NT), dim3(256), (size_t)K * sizeof(float), st,
                     ctx->pdl, q));
  MmaParams p = {};
  int t = 0;
  TcEncodeTiledFn encode = tc_tensor_map_encoder();
  HB_REQUIRE(encode != nullptr, "bitlinear (batched): the driver has no cuTensorMapEncodeTiled");
  for (int s = 0; s < nseg; ++s) {
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_packed), segs[s].d_scale,
                segs[s].d_residual, segs[s].d_y, segs[s].d_acc, segs[s].N, t};
    t += (segs[s].N + kMmaRows - 1) / kMmaRows;
    HB_REQUIRE((reinterpret_cast<uintptr_t>(segs[s].d_packed) & 15) == 0,
               "bitlinear (batched): packed weights must be 16-byte aligned");
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 4), (cuuint64_t)segs[s].N};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 4)};  // bytes between rows
    const cuuint32_t box[2] = {(cuuint32_t)(kChunkGroups * 32), (cuuint32_t)kMmaRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = encode(&p.tmap[s], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                               const_cast<void*>(segs[s].d_packed), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    HB_REQUIRE(rc == CUDA_SUCCESS, "bitlinear (batched): cuTensorMapEncodeTiled failed (%d)",
               (int)rc);
  }
  p.nseg = nseg;
  p.K = K;
  p.M = M;
  p.part = reinterpret_cast<int32_t*>(base + kScratchSplitK);
  p.tickets = ctx->d_tickets;
  p.xq = xq;
  p.d = d;
  p.sumq = sumq;
  p.status = ctx->d_status;
  return NT == 64 ? bl_mma_launch<64>(ctx, p, t, st) : bl_mma_launch<128>(ctx, p, t, st);
}
