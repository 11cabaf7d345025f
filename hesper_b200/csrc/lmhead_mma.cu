// lmhead_mma.cu -- batched (16..64 tokens) LM head on the 5th-generation tensor cores.
//
// logits[m][v] = sum_k table[v][k] * xn[m][k] with the 16-bit table (bf16 or f16, [V][K], the
// tied embedding of Hesper/Models/BitNet.lean:456) and f32 activations, optional final RMSNorm
// in front and the greedy argmax (first strict maximum, Hesper/Inference/Sampling.lean:74)
// behind.  The batch-1 kernel streams the table once per 8 tokens and is FMA-bound from 16
// tokens on; here the table is streamed ONCE and the contraction runs as tcgen05.mma
// kind::f16 with f32 accumulators in tensor memory.
//
// Keeping f32-activation accuracy on a 16-bit tensor-core path: each activation is split as
// x = hi + lo with hi = round16(x), lo = round16(x - hi).  Products of 16-bit values are exact
// in the f32 accumulator, so the logit error is that of dropping x - hi - lo (2^-17 relative
// for bf16, 2^-22 for f16) plus the accumulation order.  hi and lo occupy token rows 0..63
// and 64..127 of one N=128 operand; the epilogue adds the two halves.
//
//   lm_split_kernel     one CTA per token: optional RMSNorm, split, and store in the
//                       shared-memory operand layout (K-major 8x16-byte core matrices), one
//                       16 KB block per 64-wide K step
//   lmhead_mma_kernel   one CTA per 128 vocabulary rows, two CTAs per SM so that one tile's
//                       epilogue overlaps the other's main loop:
//     warp 0  producer: table tile [128 rows x 64 el] per step by ONE 2-D tensor-map TMA
//             (128-byte swizzle, consumed by the tensor core as it lands) + one bulk copy of
//             the 16 KB activation block;
//     warp 1  one thread issues 4 MMAs (M=128, N=128, K=16) per step; tcgen05.commit frees
//             the stage;
//     warps 2-5  epilogue: tcgen05.ld of hi and lo columns, add, optional logits store,
//             per-token argmax over the tile's 128 rows (redux + ballot), then one
//             atomicMax of the ordered (value,row) key per token.
// Every mbarrier wait is bounded; on expiry the kernel still releases its tensor memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tcgen05.cuh"

namespace hb {

constexpr int kLmRows = 128;      // vocabulary rows per CTA = MMA M
constexpr int kLmTokens = 64;     // token slots; the operand holds 2 x 64 rows (hi, lo)
constexpr int kLmN = 2 * kLmTokens;
constexpr int kLmKStep = 64;      // elements per pipeline step = 128 bytes of a table row
constexpr int kLmStages = 3;      // stages of a CTA that shares its SM with a second one
constexpr int kLmMaxStages = 6;   // stages of a CTA alone on its SM (few row tiles)
constexpr int kLmABytes = kLmRows * kLmKStep * 2;  // 16 KB
constexpr int kLmBBytes = kLmN * kLmKStep * 2;     // 16 KB
constexpr int kLmCtrl = 4096;     // barriers, tensor-memory slot, per-warp argmax keys
constexpr int kLmThreads = 192;

struct LmSplitParams {
  const float* x;      // [M][K]
  const float* gamma;  // nullable
  float eps;
  int K, M, dtype;     // dtype 0 = bf16, 1 = f16
  int single;          // 0: hi rows 0..63, lo rows 64..127 of each block; else only the rounded
                       // value, `single` token rows per block (64, 128 or 256)
  uint8_t* xb;         // [K/64][16 KB] operand blocks
  // optional step in front: x' = pre_base + rmsnorm(x) * pre_gamma, written to pre_out and
  // used as the row from there on (K <= 10240, 16-byte aligned arrays)
  const float* pre_base;
  const float* pre_gamma;
  float* pre_out;
  // f16 staging only: the row is divided by a power of two s that brings its largest magnitude
  // into [2^13, 2^14) -- f16 has 5 exponent bits, an activation above 65504 would round to
  // infinity and one below 6e-5 lose bits -- and s is stored here for the product's epilogue
  float* rowscale;     // nullable [M]
};

struct LmMmaParams {
  CUtensorMap tmap;    // table as [V rows][K elements of 2 bytes], boxes of 128 rows x 64
  const uint8_t* xb;
  float* logits;       // nullable [M][V]
  const float* residual;  // nullable [M][V], added to what is stored in `logits`
  unsigned long long* keys;  // nullable [M]
  long V;
  long ldy;            // token stride of logits / residual (>= V)
  int K, M;
  int stages;          // kLmStages or kLmMaxStages
  int table_constant;  // the table is not written by kernels of this stream (weights proper)
  const float* rowscale;  // nullable [M]: factor the staging divided each token's row by
  uint32_t idesc;
  uint32_t* status;
};

__device__ __forceinline__ uint16_t round16(float v, int dtype) {
  return dtype == 0 ? __bfloat16_as_ushort(__float2bfloat16_rn(v))
                    : __half_as_ushort(__float2half_rn(v));
}
__device__ __forceinline__ float widen16(uint16_t h, int dtype) {
  return dtype == 0 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
}

__global__ void __launch_bounds__(256) lm_split_kernel(const __grid_constant__ LmSplitParams p) {
  __shared__ double red[8];
  __shared__ float redf[8];
  pdl_trigger();
  // norm weights are constants of the model: into L1 before the wait on the previous kernel
  for (int i = threadIdx.x * 32; i < p.K; i += 256 * 32) {
    if (p.gamma) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gamma + i));
    if (p.pre_gamma) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.pre_gamma + i));
  }
  pdl_wait();
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K;
  // 8 consecutive k of token row `row` -> their 16 bytes in the operand block
  const size_t blk_bytes = p.single ? (size_t)p.single * 128 : (size_t)kLmBBytes;
  auto dst = [&](int row, int k) {
    return p.xb + (size_t)(k >> 6) * blk_bytes + (size_t)(row >> 3) * 1024 +
           (size_t)((k & 63) >> 3) * 128 + (size_t)(row & 7) * 16;
  };
  if (m >= p.M) {
    for (int k = tid * 8; k < K; k += 256 * 8) {
      *reinterpret_cast<uint4*>(dst(m, k)) = make_uint4(0, 0, 0, 0);
      if (!p.single) *reinterpret_cast<uint4*>(dst(kLmTokens + m, k)) = make_uint4(0, 0, 0, 0);
    }
    return;
  }
  const float* xg = p.x + (size_t)m * K;
  float inv_s = 1.f;  // 1 / row scale, set before the first emit
  // block-wide: the power of two that brings `amax` into [2^13, 2^14); stores it, returns 1/s
  auto row_scale = [&](float amax) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 8));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (lane == 0) redf[warp] = amax;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, redf[i]);
    int e = 13;  // an all-zero (or non-finite) row keeps s = 1
    if (amax > 0.f && amax <= 3.0e38f) e = min(max(ilogbf(amax), -100), 120);
    if (tid == 0) p.rowscale[m] = ldexpf(1.f, e - 13);
    return ldexpf(1.f, 13 - e);
  };
  auto emit = [&](int k, const float (&vin)[8]) {
    uint32_t hi[4], lo[4];
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = vin[e] * inv_s;  // exact: a power of two
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint16_t h[2], l[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        h[e] = round16(v[2 * j + e], p.dtype);
        l[e] = round16(__fsub_rn(v[2 * j + e], widen16(h[e], p.dtype)), p.dtype);
      }
      hi[j] = (uint32_t)h[0] | ((uint32_t)h[1] << 16);
      lo[j] = (uint32_t)l[0] | ((uint32_t)l[1] << 16);
    }
    *reinterpret_cast<uint4*>(dst(m, k)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    if (!p.single)
      *reinterpret_cast<uint4*>(dst(kLmTokens + m, k)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  };
  constexpr int kHeld = 5;  // 8-element groups a thread keeps in registers: K <= 10240
  const bool aligned =
      ((reinterpret_cast<uintptr_t>(xg) | reinterpret_cast<uintptr_t>(p.gamma)) & 15) == 0;
  if (K <= kHeld * 2048 && aligned) {
    // the row is read once and stays in registers between the sum of squares and the rounding
    float v[kHeld][8];
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int k = tid * 8 + i * 2048;
      const bool in = k < K;
      const float4 a = in ? *reinterpret_cast<const float4*>(xg + k) : make_float4(0, 0, 0, 0);
      const float4 b = in ? *reinterpret_cast<const float4*>(xg + k + 4) : make_float4(0, 0, 0, 0);
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
      v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
    }
    auto row_rinv = [&]() {  // 1 / rms of the row held in v (block-wide)
      double ss = 0.0;
#pragma unroll
      for (int i = 0; i < kHeld; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += (double)v[i][e] * v[i][e];
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = 0.0;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += red[i];
      __syncthreads();  // red may be written again
      return (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
    };
    if (p.pre_gamma) {
      // the addend is fetched before the reduction, so that it shares the row's trip to L2
      const float* bg = p.pre_base + (size_t)m * K;
      float* og = p.pre_out + (size_t)m * K;
      float b[kHeld][8];
#pragma unroll
      for (int i = 0; i < kHeld; ++i) {
        const int k = tid * 8 + i * 2048;
        const bool in = k < K;
        const float4 ba = in ? *reinterpret_cast<const float4*>(bg + k) : make_float4(0, 0, 0, 0);
        const float4 bb = in ? *reinterpret_cast<const float4*>(bg + k + 4) : make_float4(0, 0, 0, 0);
        b[i][0] = ba.x; b[i][1] = ba.y; b[i][2] = ba.z; b[i][3] = ba.w;
        b[i][4] = bb.x; b[i][5] = bb.y; b[i][6] = bb.z; b[i][7] = bb.w;
      }
      const float r1 = row_rinv();
#pragma unroll
      for (int i = 0; i < kHeld; ++i) {
        const int k = tid * 8 + i * 2048;
        if (k >= K) continue;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(p.pre_gamma + k));
        const float4 gb = __ldg(reinterpret_cast<const float4*>(p.pre_gamma + k + 4));
        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v[i][e] = __fadd_rn(b[i][e], __fmul_rn(__fmul_rn(v[i][e], r1), g[e]));
        *reinterpret_cast<float4*>(og + k) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
        *reinterpret_cast<float4*>(og + k + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
      }
    }
    if (p.gamma) {
      const float rinv = row_rinv();
#pragma unroll
      for (int i = 0; i < kHeld; ++i) {
        const int k = tid * 8 + i * 2048;
        if (k >= K) continue;
        const float4 ga = __ldg(reinterpret_cast<const float4*>(p.gamma + k));
        const float4 gb = __ldg(reinterpret_cast<const float4*>(p.gamma + k + 4));
        const float g[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __fmul_rn(__fmul_rn(v[i][e], rinv), g[e]);
      }
    }
    if (p.rowscale) {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < kHeld; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[i][e]));  // rows past K hold zeros
      inv_s = row_scale(amax);
    }
#pragma unroll
    for (int i = 0; i < kHeld; ++i) {
      const int k = tid * 8 + i * 2048;
      if (k < K) emit(k, v[i]);
    }
    return;
  }
  float rinv = 1.f;
  if (p.gamma) {
    double ss = 0.0;
    for (int k = tid; k < K; k += 256) {
      const float v = xg[k];
      ss += (double)v * v;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += red[i];
    rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
  }
  if (p.rowscale) {
    float amax = 0.f;
    for (int k = tid; k < K; k += 256)
      amax = fmaxf(amax, fabsf(p.gamma ? __fmul_rn(__fmul_rn(xg[k], rinv), p.gamma[k]) : xg[k]));
    inv_s = row_scale(amax);
  }
  for (int k = tid * 8; k < K; k += 256 * 8) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e)
      v[e] = p.gamma ? __fmul_rn(__fmul_rn(xg[k + e], rinv), p.gamma[k + e]) : xg[k + e];
    emit(k, v);
  }
}

// kind::f16 with both operands through shared-memory descriptors.
__device__ __forceinline__ void lm_umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kLmThreads, 2)
    lmhead_mma_kernel(const __grid_constant__ LmMmaParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nsteps = p.K / kLmKStep;
  const int S = p.stages;
  const long row0 = (long)blockIdx.x * kLmRows;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem);   // [kLmStages] table box + activations
  uint64_t* empty = full + kLmMaxStages;                 // [stages] MMAs of the stage retired
  uint64_t* done = empty + kLmMaxStages;                 // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  unsigned long long* wkeys = reinterpret_cast<unsigned long long*>(smem + 1024);  // [4][64]
  uint8_t* stg = smem + kLmCtrl;  // per stage: A (16 KB, swizzled) then B (16 KB)

  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 2);  // one arrival with the table bytes, one with the activation bytes
      mbar_init(&empty[i], 1);
    }
    mbar_init(done, 1);
    fence_mbar_init();
  }
  if (warp == 1) {  // 128 columns: the 128 x 128 f32 accumulator
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(
        smem_u32(tmem_slot)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_before_sync();
  __syncthreads();
  tc_after_sync();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (warp == 0) {
    // ================= producer =============================================================
    const uint64_t pol = policy_evict_first();
    auto issue_a = [&](int ks) {
      const int st = ks % S;
      mbar_arrive_expect_tx(&full[st], kLmABytes);
      tc_tma_box_2d(stg + (size_t)st * (kLmABytes + kLmBBytes), &p.tmap, ks * kLmKStep, (int)row0,
                 &full[st], pol);
    };
    auto issue_b = [&](int ks) {
      const int st = ks % S;
      mbar_arrive_expect_tx(&full[st], kLmBBytes);
      bulk_g2s(stg + (size_t)st * (kLmABytes + kLmBBytes) + kLmABytes,
               p.xb + (size_t)ks * kLmBBytes, kLmBBytes, &full[st]);
    };
    const int pre = min(S, nsteps);
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&p.tmap))
                   : "memory");
      // a constant table (the LM head) can be fetched before the dependency resolves; a table
      // that kernels of this stream write cannot
      if (p.table_constant)
        for (int ks = 0; ks < pre; ++ks) issue_a(ks);
    }
    pdl_trigger();
    pdl_wait();  // the split activations come from the kernel before this one
    if (lane == 0)
      for (int ks = 0; ks < pre; ++ks) {
        if (!p.table_constant) issue_a(ks);
        issue_b(ks);
      }
    for (int ks = pre; ks < nsteps; ++ks) {
      ok = tc_wait(ok, &empty[ks % S], (uint32_t)(((ks / S) - 1) & 1), p.status);
      if (lane == 0 && ok) {
        issue_a(ks);
        issue_b(ks);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer ===========================================================
    for (int ks = 0; ks < nsteps; ++ks) {
      const int st = ks % S;
      ok = tc_wait(ok, &full[st], (uint32_t)((ks / S) & 1), p.status);
      if (lane == 0) {
        tc_after_sync();
        const uint32_t abase = smem_u32(stg + (size_t)st * (kLmABytes + kLmBBytes));
        const uint32_t bbase = abase + kLmABytes;
#pragma unroll
        for (int j = 0; j < kLmKStep / 16; ++j)  // K = 16 elements = 32 bytes per instruction
          lm_umma_f16(tmem, tc_smem_desc(abase + j * 32, 0, 1024, 2),
                      tc_smem_desc(bbase + j * 256, 128, 1024, 0), p.idesc,
                      (ks > 0 || j > 0) ? 1u : 0u);
        tc_commit(&empty[st]);
      }
      __syncwarp();
    }
    if (lane == 0) tc_commit(done);
  }
  // ================= epilogue (warps 2..5) ====================================================
  if (warp >= 2) {
    ok = tc_wait(true, done, 0, p.status);
    tc_after_sync();
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const long row = row0 + q * 32 + lane;
    const bool row_ok = row < p.V;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
    unsigned long long* mykeys = wkeys + (warp - 2) * kLmTokens;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      if (half * 32 >= p.M) {
        if (lane < 32) mykeys[half * 32 + lane] = 0ull;
        continue;
      }
      uint32_t hi[32], lo[32];
      HB_TMEM_LD32(hi, lane_addr + (uint32_t)(half * 32));
      HB_TMEM_LD32(lo, lane_addr + (uint32_t)(kLmTokens + half * 32));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      unsigned long long mine = 0ull;  // lane t keeps the key of token half*32 + t
      // lane t fetches token half*32 + t's row scale (f16 staging), a shuffle hands it around
      const float my_rs =
          (p.rowscale && half * 32 + lane < p.M) ? __ldcg(p.rowscale + half * 32 + lane) : 1.f;
#pragma unroll
      for (int t = 0; t < 32; ++t) {
        const int m = half * 32 + t;
        float v = __fadd_rn(__uint_as_float(hi[t]), __uint_as_float(lo[t]));
        v *= __shfl_sync(0xffffffffu, my_rs, t);  // undo the staging's row scale (exact)
        if (m < p.M && row_ok && p.logits && ok) {
          const size_t o = (size_t)m * p.ldy + (size_t)(row);
          p.logits[o] = p.residual ? __fadd_rn(v, p.residual[o]) : v;
        }
        if (!p.keys) continue;  // plain product: no argmax
        uint32_t u = __float_as_uint(v);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // monotone map float -> uint
        if (!(v == v) || !row_ok) u = 0u;                  // NaN and padding rows never win
        const uint32_t best = __reduce_max_sync(0xffffffffu, u);
        const uint32_t who = __ballot_sync(0xffffffffu, u == best);
        if (lane == t) {
          const uint32_t first_row = (uint32_t)(row0 + q * 32) + (uint32_t)(__ffs(who) - 1);
          mine = best ? (((unsigned long long)best << 32) |
                         (unsigned long long)(0xFFFFFFFFu - first_row))
                      : 0ull;
        }
      }
      mykeys[half * 32 + lane] = mine;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
    if (warp == 2 && p.keys && ok) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int m = lane + 32 * i;
        if (m < p.M) {
          unsigned long long k = wkeys[m];
#pragma unroll
          for (int w = 1; w < 4; ++w) {
            const unsigned long long o = wkeys[w * kLmTokens + m];
            k = o > k ? o : k;
          }
          if (k) atomicMax(&p.keys[m], k);
        }
      }
    }
  }
  tc_before_sync();
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmem));
}

}  // namespace hb

using namespace hb;

// x[M][K] (M <= 64) -> hi/lo 16-bit operand blocks in the context scratch, optional RMSNorm.
// single = 64, 128 or 256: only the rounded value (no lo term), that many token rows per
// 64-wide K block (M <= single).
int hb_gemm16_split(hb200_ctx* ctx, int dtype, int K, const float* d_x, int M,
                    const float* d_rms_gamma, float rms_eps, int single, cudaStream_t st) {
  return hb_gemm16_split_pre(ctx, dtype, K, d_x, M, nullptr, nullptr, nullptr, d_rms_gamma,
                             rms_eps, single, st);
}

// The same with x' = d_pre_base + rmsnorm(d_x) * d_pre_gamma computed first (written to
// d_pre_out and staged); d_pre_gamma null: no such step.
int hb_gemm16_split_pre(hb200_ctx* ctx, int dtype, int K, const float* d_x, int M,
                        const float* d_pre_base, const float* d_pre_gamma, float* d_pre_out,
                        const float* d_rms_gamma, float rms_eps, int single, cudaStream_t st) {
  if (d_pre_gamma) {
    HB_REQUIRE(d_pre_base && d_pre_out && K <= 10240 &&
                   ((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_rms_gamma) |
                     reinterpret_cast<uintptr_t>(d_pre_base) |
                     reinterpret_cast<uintptr_t>(d_pre_gamma) |
                     reinterpret_cast<uintptr_t>(d_pre_out)) & 15) == 0,
               "batched 16-bit product: pre-step needs K <= 10240 and 16-byte aligned arrays");
  }
  HB_REQUIRE(single == 0 || single == 64 || single == 128 || single == 256,
             "batched 16-bit product: %d token rows per block", single);
  const size_t xb_bytes = (size_t)(K / kLmKStep) * (single ? (size_t)single * 128 : (size_t)kLmBBytes);
  HB_REQUIRE(kScratchLmSplit + xb_bytes <= kScratchSplitK,
             "batched 16-bit product: K=%d needs %zu bytes of activation scratch", K, xb_bytes);
  HB_REQUIRE(M >= 1 && M <= (single ? single : kLmTokens), "batched 16-bit product: M=%d", M);
  uint8_t* xb = static_cast<uint8_t*>(ctx->d_scratch) + kScratchLmSplit;
  float* rowscale = dtype == 1 ? reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->d_scratch) +
                                                         kScratchRowScale)
                               : nullptr;  // bf16 has the exponent range of f32
  LmSplitParams sp = {d_x, d_rms_gamma, rms_eps, K, M, dtype, single, xb,
                      d_pre_base, d_pre_gamma, d_pre_out, rowscale};
  HB_CUDA(launch_pdl(lm_split_kernel, dim3(single ? single : kLmTokens), dim3(256), 0, st,
                     ctx->pdl, sp));
  return HB200_OK;
}

// y[m*ldy + v] = sum_k table[v][k] * x[m][k] (+ residual[m*ldy + v]) for the activations
// staged by hb_gemm16_split; d_y nullable, d_keys nullable (argmax keys, atomicMax like the batch-1
// LM head so that the finishing kernel is shared).
int hb_gemm16_mma(hb200_ctx* ctx, const void* d_table, int dtype, long V, int K, int M,
                  float* d_y, const float* d_residual, long ldy, unsigned long long* d_keys,
                  int table_constant, cudaStream_t st) {
  HB_REQUIRE(V >= 1 && V < (1l << 31), "batched 16-bit product: bad row count");
  uint8_t* xb = static_cast<uint8_t*>(ctx->d_scratch) + kScratchLmSplit;
  LmMmaParams p = {};
  TcEncodeTiledFn encode = tc_tensor_map_encoder();
  HB_REQUIRE(encode != nullptr, "batched 16-bit product: the driver has no cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)V};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kLmKStep, (cuuint32_t)kLmRows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc =
      encode(&p.tmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(d_table), dims, strides,
             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  HB_REQUIRE(rc == CUDA_SUCCESS, "batched 16-bit product: cuTensorMapEncodeTiled failed (%d)",
             (int)rc);
  p.xb = xb;
  p.logits = d_y;
  p.residual = d_residual;
  p.keys = d_keys;
  p.rowscale = dtype == 1 ? reinterpret_cast<const float*>(static_cast<const uint8_t*>(ctx->d_scratch) +
                                                           kScratchRowScale)
                          : nullptr;
  p.V = V;
  p.ldy = ldy;
  p.K = K;
  p.M = M;
  p.table_constant = table_constant;
  // instruction descriptor of kind::f16: D = f32, A and B of the table's type, both K-major
  const uint32_t fmt = dtype == 0 ? 1u : 0u;  // 1 = bf16, 0 = f16
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kLmN >> 3) << 17) |
            ((uint32_t)(kLmRows >> 4) << 24);
  p.status = ctx->d_status;
  {
    const int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(lmhead_mma_kernel),
                                (size_t)(kLmCtrl + kLmMaxStages * (kLmABytes + kLmBBytes)));
    if (rc != HB200_OK) return rc;
  }
  const long ntiles = (V + kLmRows - 1) / kLmRows;
  // few row tiles: every CTA has an SM to itself, so it takes the deeper ring (192 KB in
  // flight) instead of sharing the SM with a CTA that does not exist
  p.stages = ntiles <= ctx->sm_count ? kLmMaxStages : kLmStages;
  const size_t smem = kLmCtrl + (size_t)p.stages * (kLmABytes + kLmBBytes);
  HB_CUDA(launch_pdl(lmhead_mma_kernel, dim3((unsigned)ntiles), dim3(kLmThreads), smem, st,
                     ctx->pdl, p));
  return HB200_OK;
}

// Batched LM head (16 <= M <= 64, K a multiple of 64).
int hb_lmhead_mma_run(hb200_ctx* ctx, const void* d_table, int dtype, long V, int K,
                      const float* d_x, int M, const float* d_rms_gamma, float rms_eps,
                      float* d_logits, unsigned long long* d_keys, cudaStream_t st) {
  ScratchUse use(ctx, st);  // the staged hi / lo activations
  const int rc = hb_gemm16_split(ctx, dtype, K, d_x, M, d_rms_gamma, rms_eps, 0, st);
  if (rc != HB200_OK) return rc;
  return hb_gemm16_mma(ctx, d_table, dtype, V, K, M, d_logits, nullptr, V, d_keys, 1, st);
}
