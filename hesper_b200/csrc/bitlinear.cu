// bitlinear.cu -- ternary (i2_s) x int8 matvec for sm_100a.
//
// What it computes is BitLinearSpec.forward (Hesper/Layers/BitLinearSpec.lean:65-91)
// on int8 activations: acc[n] = sum_k t[n,k]*q[k] exactly in int32, then
// y = ((float)acc*d)*s (+residual).  The reference's kernels for the same layer
// are fusedBitLinearM1Kernel and its residual / RMSNorm / gate-up variants
// (Hesper/Layers/BitLinear.lean:297,361,447,553).
//
// How it runs on B200:
//   * the rows are cut into tiles of RT rows; tiles are split evenly over the
//     grid (one CTA per SM) and dealt round-robin to the warps of a CTA.  Every
//     warp is its own streaming engine: lane 0 pulls a tile global->shared with a
//     1-D TMA bulk copy completed on a per-warp mbarrier ring, so no CTA-wide
//     barrier sits in the streaming loop;
//   * the weight prefetch is issued BEFORE griddepcontrol.wait: under programmatic
//     dependent launch the bytes of this layer are in flight while the previous
//     kernel of the decode step is still finishing.  A launch keeps to at most
//     half of an SM's registers and shared memory so that two consecutive layers
//     are resident together;
//   * meanwhile the whole CTA runs the activation prologue (optional RMSNorm,
//     absmax, int8 quantisation) into shared memory, laid out so that the four
//     2-bit planes of a packed word meet their activations as four dp4a operands;
//   * unpacking is four ANDs per 16 weights: plane p of word w is w & (3 << 2p)
//     per byte, i.e. the code scaled by 4^p, which dp4a.u32.s32 multiplies
//     directly; the scale is shifted out once per row and sum(q) is subtracted
//     once (value = code - 1);
//   * a transposing shuffle reduction turns the per-lane row partials of a tile
//     into row sums with a handful of shuffles.
// At batch 1 the kernel is as much instruction-issue- and latency-bound as it is
// bandwidth-bound (a 4.4 MB matrix is 0.7 us of HBM time), which is why the
// prologue is kept to a few dozen instructions per thread and every load that
// does not depend on the previous kernel is hoisted above the dependency wait.
#include <stdio.h>

#include "common.cuh"

namespace hb {


constexpr int kBLMaxSeg = 4;

struct BLSeg {
  const uint8_t* w;
  const float* scale;
  const float* residual;
  float* y;
  int32_t* acc;
  int N;
  int tile0;  // first tile of this segment
};

struct BLParams {
  BLSeg seg[kBLMaxSeg];
  int nseg;
  int gateup;  // 1: seg[0] = gate, seg[1] = up, fused ReLU^2 GLU epilogue
  int ntiles;  // tiles over all segments (a tile never straddles two segments)
  int K;
  int M;       // tokens
  int stages;  // ring depth per warp
  const float* x;  // [M][K]
  const float* gamma;
  float eps;
  float* act_scale;  // nullable [M]
  uint32_t* status;
};

// Sum of NS per-lane partials across the warp (NS = 2, 4 or 8).  Each of the
// first log2(NS) butterfly stages halves the number of live values, the rest
// are plain exchanges; afterwards every lane holds the complete sum of slot
// lane >> (5 - log2(NS)).
template <int NS>
__device__ __forceinline__ int transpose_reduce(const int (&a)[NS], int lane) {
  int v[NS];
#pragma unroll
  for (int i = 0; i < NS; ++i) v[i] = a[i];
  int bit = 16;
#pragma unroll
  for (int n = NS; n > 1; n >>= 1) {
    const bool hi = lane & bit;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const int send = hi ? v[i] : v[i + n / 2];
      const int keep = hi ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
    }
    bit >>= 1;
  }
#pragma unroll
  for (; bit >= 1; bit >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], bit);
  return v[0];
}

// WPL : packed words per lane per K-chunk (a chunk is 32*WPL words = 512*WPL weights)
// MT  : tokens sharing one pass over the weights
// RT  : rows per tile (a gate/up tile holds RT gate rows and RT up rows)
// GU  : fused gate/up ReLU^2 GLU
template <int WPL, int MT, int RT, bool GU>
struct BLCfg {
  static constexpr int kThreads = MT == 1 ? 384 : 256;
  static constexpr int kWarps = kThreads / 32;
  static constexpr int kSlots = GU ? 2 * RT : RT;  // accumulators per tile
  static constexpr int kMinBlocks = MT == 1 ? 2 : 1;
};

template <int WPL, int MT, int RT, bool GU>
__global__ void __launch_bounds__(BLCfg<WPL, MT, RT, GU>::kThreads,
                                  BLCfg<WPL, MT, RT, GU>::kMinBlocks)
    bitlinear_kernel(const __grid_constant__ BLParams p) {
  using Cfg = BLCfg<WPL, MT, RT, GU>;
  constexpr int kThreads = Cfg::kThreads, kWarps = Cfg::kWarps, kSlots = Cfg::kSlots;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K;
  const int words = K >> 4;     // packed u32 per row
  const int rowbytes = K >> 2;  // packed bytes per row
  const int PS = words + 8;     // plane stride of the int8 activations (bank spread)
  const int S = p.stages;
  const int stage_bytes = kSlots * rowbytes;

  // shared memory carve-up (bl_smem_bytes on the host mirrors it)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [warps][S]
  size_t off = (size_t)kWarps * S * sizeof(uint64_t);
  off = (off + 127) & ~size_t(127);
  double* red_f64 = reinterpret_cast<double*>(smem + off);  // [MT][16]
  off += MT * 16 * sizeof(double);
  uint32_t* red_u32 = reinterpret_cast<uint32_t*>(smem + off);  // [MT][16]
  off += MT * 16 * sizeof(uint32_t);
  int* red_i32 = reinterpret_cast<int*>(smem + off);  // [MT][16]
  off += MT * 16 * sizeof(int);
  float* tok_d = reinterpret_cast<float*>(smem + off);  // [MT] activation scales
  off += 8 * sizeof(float);
  off = (off + 127) & ~size_t(127);
  float* xf = reinterpret_cast<float*>(smem + off);  // [K] staging of one token
  off += (size_t)K * sizeof(float);
  uint32_t* xq = reinterpret_cast<uint32_t*>(smem + off);  // [MT][4 planes][PS]
  off += (size_t)MT * 4 * PS * sizeof(uint32_t);
  off = (off + 127) & ~size_t(127);
  uint8_t* wstage = smem + off + (size_t)warp * S * stage_bytes;
  uint64_t* mybar = bars + warp * S;

  // tiles [t0, t1) belong to this CTA; warp w takes t0+w, t0+w+kWarps, ...
  const int G = gridDim.x;
  const int t0 = (int)(((long long)blockIdx.x * p.ntiles) / G);
  const int t1 = (int)(((long long)(blockIdx.x + 1) * p.ntiles) / G);

  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&mybar[s], 1);
    fence_mbar_init();
  }
  if (tid < 16 * MT) {  // unused warp slots of the reduction scratch must read as 0
    red_f64[tid] = 0.0;
    red_u32[tid] = 0u;
    red_i32[tid] = 0;
  }
  __syncwarp();
  const uint64_t pol = policy_evict_first();

  // tile -> (segment, first row, live rows)
  auto tile_at = [&](int t, int& seg, int& row, int& nr) {
    seg = 0;
    if (!GU) {
#pragma unroll
      for (int s = 1; s < kBLMaxSeg; ++s)
        if (s < p.nseg && t >= p.seg[s].tile0) seg = s;
    }
    row = (t - p.seg[seg].tile0) * RT;
    nr = min(RT, p.seg[seg].N - row);
  };

  // Ring bookkeeping is warp-uniform: every lane tracks the cursors, lane 0 issues.
  // The warp's tile number i (counted over all passes) lives in stage i % S and
  // completes phase (i / S) & 1 of that stage's mbarrier.
  int issued = 0, consumed = 0, tprod = t0 + warp;
  auto produce = [&]() {
    int seg, row, nr;
    tile_at(tprod, seg, row, nr);
    if (lane == 0) {
      const int stage = issued % S;
      uint8_t* dst = wstage + (size_t)stage * stage_bytes;
      const uint32_t bytes = (uint32_t)nr * rowbytes;
      if (!GU) {
        mbar_arrive_expect_tx(&mybar[stage], bytes);
        bulk_g2s_stream(dst, p.seg[seg].w + (size_t)row * rowbytes, bytes, &mybar[stage], pol);
      } else {
        mbar_arrive_expect_tx(&mybar[stage], 2 * bytes);
        bulk_g2s_stream(dst, p.seg[0].w + (size_t)row * rowbytes, bytes, &mybar[stage], pol);
        bulk_g2s_stream(dst + (size_t)RT * rowbytes, p.seg[1].w + (size_t)row * rowbytes, bytes,
                        &mybar[stage], pol);
      }
    }
    tprod += kWarps;
    ++issued;
  };

  // ---- weight prefetch and every other load that does not depend on the
  //      previous kernel --------------------------------------------------------
  while (issued < S && tprod < t1) produce();
  float wscale[GU ? 2 : kBLMaxSeg];
#pragma unroll
  for (int s = 0; s < (GU ? 2 : kBLMaxSeg); ++s)
    wscale[s] = s < p.nseg ? __ldg(p.seg[s].scale) : 0.f;
  const int M = p.M;
  const float* const xbase = p.x;
  const float* const gamma = p.gamma;
  // the norm weights are constants of the model: pull their lines into L1 now, so that the
  // loads after the sum-of-squares reduction do not pay a second trip to L2
  if (gamma)
    for (int i = tid * 32; i < K; i += kThreads * 32)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(gamma + i));
  pdl_trigger();
  pdl_wait();  // activations (and residuals) come from the previous kernel

  const int nchunks = (words + 32 * WPL - 1) / (32 * WPL);
  const int nvec = K >> 2;

  for (int m0 = 0; m0 < M; m0 += MT) {
    // ---- activation prologue: RMSNorm (optional), absmax, int8 --------------
    __syncthreads();  // scratch initialised / all warps done with the previous xq
#pragma unroll 1
    for (int mt = 0; mt < MT; ++mt) {
      const int m = m0 + mt;
      uint32_t* xqm = xq + (size_t)mt * 4 * PS;
      if (m >= M) {  // padding token: zeros
        for (int i = tid; i < 4 * PS; i += kThreads) xqm[i] = 0u;
        if (lane == 0) {
          red_i32[mt * 16 + warp] = 0;
          if (warp == 0) tok_d[mt] = 0.f;
        }
        continue;
      }
      const float4* xg = reinterpret_cast<const float4*>(xbase + (size_t)m * K);
      float4* xs = reinterpret_cast<float4*>(xf);
      float amax = 0.f;
      if (gamma) {
        double ss = 0.0;
        for (int i = tid; i < nvec; i += kThreads) {
          const float4 v = __ldcg(xg + i);
          xs[i] = v;
          ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) red_f64[mt * 16 + warp] = ss;
        __syncthreads();
        ss = 0.0;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) ss += red_f64[mt * 16 + i];
        const float rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
        const float4* gg = reinterpret_cast<const float4*>(gamma);
        for (int i = tid; i < nvec; i += kThreads) {
          float4 v = xs[i];
          const float4 g = __ldg(gg + i);
          v.x = __fmul_rn(__fmul_rn(v.x, rinv), g.x);
          v.y = __fmul_rn(__fmul_rn(v.y, rinv), g.y);
          v.z = __fmul_rn(__fmul_rn(v.z, rinv), g.z);
          v.w = __fmul_rn(__fmul_rn(v.w, rinv), g.w);
          xs[i] = v;
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
      } else {
        for (int i = tid; i < nvec; i += kThreads) {
          const float4 v = __ldcg(xg + i);
          xs[i] = v;
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
      }
      // non-negative floats order like their bit patterns: one redux per warp
      const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
      if (lane == 0) red_u32[mt * 16 + warp] = wmax;
      __syncthreads();
      {
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
          const uint4 a = *reinterpret_cast<const uint4*>(red_u32 + mt * 16 + i);
          mx = max(mx, max(max(a.x, a.y), max(a.z, a.w)));
        }
        amax = __uint_as_float(mx);
      }
      const float d = __fdiv_rn(amax, 127.0f);
      const float inv = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
      int sumq = 0;
      for (int i = tid; i < nvec; i += kThreads) {
        const float4 v = xs[i];
        const int q0 = __float2int_rn(__fmul_rn(v.x, inv));
        const int q1 = __float2int_rn(__fmul_rn(v.y, inv));
        const int q2 = __float2int_rn(__fmul_rn(v.z, inv));
        const int q3 = __float2int_rn(__fmul_rn(v.w, inv));
        sumq += (q0 + q1) + (q2 + q3);
        // float4 i = elements 4i..4i+3: group g = i/32, plane s, byte-quad wi
        const int g = i >> 5, s = (i >> 3) & 3, wi = i & 7;
        const uint32_t pk = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) |
                            ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)q3 << 24);
        xqm[s * PS + g * 8 + wi] = pk;
      }
      sumq = __reduce_add_sync(0xffffffffu, sumq);
      if (lane == 0) {
        red_i32[mt * 16 + warp] = sumq;
        if (warp == 0) {
          tok_d[mt] = d;
          if (p.act_scale && blockIdx.x == 0) p.act_scale[m] = d;
        }
      }
    }
    __syncthreads();

    // ---- streaming main loop (per warp) --------------------------------------
    // Token groups after the first stream the weights again (from L2 by then).
    if (m0 > 0) {
      tprod = t0 + warp;
      for (int n = 0; n < S && tprod < t1; ++n) produce();
    }
    int sumq[MT];
    float dtok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      int sq = 0;
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const int4 a = *reinterpret_cast<const int4*>(red_i32 + mt * 16 + i);
        sq += (a.x + a.y) + (a.z + a.w);
      }
      sumq[mt] = sq;
      dtok[mt] = tok_d[mt];
    }

    for (int t = t0 + warp; t < t1; t += kWarps) {
      const int stage = consumed % S;
      const uint32_t parity = (uint32_t)((consumed / S) & 1);
      int seg, row, nr;
      tile_at(t, seg, row, nr);
      mbar_wait(&mybar[stage], parity, p.status);
      const uint32_t* ws = reinterpret_cast<const uint32_t*>(wstage + (size_t)stage * stage_bytes);

      // Rows beyond `nr` of a partial tile are computed on whatever the stage
      // holds and then dropped: integer garbage is harmless and the loop stays
      // branch-free.
      int acc[MT][kSlots];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < kSlots; ++r) acc[mt][r] = 0;

#pragma unroll 1
      for (int ch = 0; ch < nchunks; ++ch) {
        uint32_t xr[MT][WPL][4];
        int jidx[WPL];
#pragma unroll
        for (int i = 0; i < WPL; ++i) {
          const int j = (ch * WPL + i) * 32 + lane;
          const bool ok = j < words;
          jidx[i] = ok ? j : (words - 1);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint32_t* xqm = xq + (size_t)mt * 4 * PS;
#pragma unroll
            for (int s = 0; s < 4; ++s) xr[mt][i][s] = ok ? xqm[s * PS + jidx[i]] : 0u;
          }
        }
#pragma unroll
        for (int r = 0; r < kSlots; ++r) {
          const uint32_t* wr = ws + r * words;
          int a0[MT], a1[MT], a2[MT], a3[MT];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) a0[mt] = a1[mt] = a2[mt] = a3[mt] = 0;
#pragma unroll
          for (int i = 0; i < WPL; ++i) {
            const uint32_t w = wr[jidx[i]];
            const uint32_t p0 = w & 0xC0C0C0C0u, p1 = w & 0x30303030u;
            const uint32_t p2 = w & 0x0C0C0C0Cu, p3 = w & 0x03030303u;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              a0[mt] = dp4a_us(p0, xr[mt][i][0], a0[mt]);
              a1[mt] = dp4a_us(p1, xr[mt][i][1], a1[mt]);
              a2[mt] = dp4a_us(p2, xr[mt][i][2], a2[mt]);
              a3[mt] = dp4a_us(p3, xr[mt][i][3], a3[mt]);
            }
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            acc[mt][r] += (a0[mt] >> 6) + (a1[mt] >> 4) + (a2[mt] >> 2) + a3[mt];
        }
      }
      __syncwarp();  // every lane has finished reading this stage
      if (tprod < t1) produce();  // refill it with the warp's tile S ahead

      // ---- reduce and store ---------------------------------------------------
      constexpr int kShift = kSlots == 8 ? 2 : (kSlots == 4 ? 3 : 4);
      const int slot = lane >> kShift;
      const bool writer = (lane & ((1 << kShift) - 1)) == 0;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = m0 + mt;
        const int total = transpose_reduce<kSlots>(acc[mt], lane) - sumq[mt];
        if (!GU) {
          if (writer && slot < nr && m < M) {
            const BLSeg& sg = p.seg[seg];
            const size_t o = (size_t)m * sg.N + row + slot;
            if (sg.acc) sg.acc[o] = total;
            float ws_ = wscale[0];
#pragma unroll
            for (int s = 1; s < kBLMaxSeg; ++s) ws_ = seg == s ? wscale[s] : ws_;
            float v = __fmul_rn(__fmul_rn((float)total, dtok[mt]), ws_);
            if (sg.residual) v = __fadd_rn(v, sg.residual[o]);
            sg.y[o] = v;
          }
        } else {
          // gate row i sits in slot i, up row i in slot RT + i: half a warp apart
          const int up = __shfl_down_sync(0xffffffffu, total, 16);
          if (writer && slot < RT && slot < nr && m < M) {
            const size_t o = (size_t)m * p.seg[0].N + row + slot;
            const float g = __fmul_rn(__fmul_rn((float)total, dtok[mt]), wscale[0]);
            const float u = __fmul_rn(__fmul_rn((float)up, dtok[mt]), wscale[1]);
            const float r = g > 0.f ? g : 0.f;
            p.seg[0].y[o] = __fmul_rn(__fmul_rn(r, r), u);
          }
        }
      }
      ++consumed;
    }
  }
}

// ---- host side ------------------------------------------------------------------

static int pick_wpl(int words) {
  int best = 8, best_pad = 1 << 30;
  for (int w = 8; w >= 4; --w) {
    const int per = 32 * w;
    const int pad = (words + per - 1) / per * per - words;
    if (pad < best_pad) {
      best_pad = pad;
      best = w;
    }
  }
  return best;
}

// Shared memory of one CTA; mirrors the carve-up at the top of the kernel.
static size_t bl_smem_bytes(int warps, int stages, int slots, int K, int MT) {
  auto up128 = [](size_t v) { return (v + 127) & ~size_t(127); };
  size_t off = up128((size_t)warps * stages * 8);
  off += (size_t)MT * 16 * (8 + 4 + 4) + 8 * 4;
  off = up128(off);
  off += (size_t)K * 4 + (size_t)MT * 4 * (K / 16 + 8) * 4;
  off = up128(off);
  return off + (size_t)warps * stages * slots * (size_t)(K / 4);
}

template <int WPL, int MT, int RT, bool GU>
static int bl_launch(hb200_ctx* ctx, BLParams& p, cudaStream_t st) {
  using Cfg = BLCfg<WPL, MT, RT, GU>;
  auto kern = bitlinear_kernel<WPL, MT, RT, GU>;
  const int grid = p.ntiles < ctx->sm_count ? p.ntiles : ctx->sm_count;
  const int tiles_per_warp = ((p.ntiles + grid - 1) / grid + Cfg::kWarps - 1) / Cfg::kWarps;
  // At batch 1 two CTAs are meant to share an SM (this layer computing while the
  // next one prefetches), so a launch takes at most half of the shared memory.
  const size_t budget = MT == 1 ? (size_t)ctx->smem_optin / 2 - 1024 : (size_t)ctx->smem_optin;
  int stages = tiles_per_warp < 4 ? tiles_per_warp : 4;
  if (stages < 1) stages = 1;
  size_t smem = 0;
  for (;; --stages) {
    smem = bl_smem_bytes(Cfg::kWarps, stages, Cfg::kSlots, p.K, MT);
    if (smem <= budget) break;
    if (stages == 1) {
      set_error("bitlinear: K=%d does not fit the shared-memory budget", p.K);
      return HB200_ERR_UNSUPPORTED;
    }
  }
  p.stages = stages;
  {
    const int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(kern), smem);
    if (rc != HB200_OK) return rc;
  }
  HB_CUDA(launch_pdl(kern, dim3(grid), dim3(Cfg::kThreads), smem, st, ctx->pdl, p));
  return HB200_OK;
}

template <int WPL, int RT, bool GU>
static int bl_dispatch_mt(hb200_ctx* ctx, BLParams& p, cudaStream_t st) {
  return p.M == 1 ? bl_launch<WPL, 1, RT, GU>(ctx, p, st) : bl_launch<WPL, 4, RT, GU>(ctx, p, st);
}

template <int RT, bool GU>
static int bl_dispatch_wpl(hb200_ctx* ctx, BLParams& p, cudaStream_t st) {
  switch (pick_wpl(p.K / 16)) {
    case 4: return bl_dispatch_mt<4, RT, GU>(ctx, p, st);
    case 5: return bl_dispatch_mt<5, RT, GU>(ctx, p, st);
    case 6: return bl_dispatch_mt<6, RT, GU>(ctx, p, st);
    case 7: return bl_dispatch_mt<7, RT, GU>(ctx, p, st);
    default: return bl_dispatch_mt<8, RT, GU>(ctx, p, st);
  }
}

// Rows per tile: 4 when that still leaves every SM a good number of tiles
// (work is dealt in whole tiles, so few tiles per SM means imbalance), else 2.
static int bl_pick_rt(const hb200_ctx* ctx, long rows_total) {
  return rows_total / 4 >= 8L * ctx->sm_count ? 4 : 2;
}

static int bl_check_common(hb200_ctx* ctx, int K, int M, const float* d_x) {
  HB_REQUIRE(ctx != nullptr, "bitlinear: null context");
  HB_REQUIRE(K > 0 && K % 128 == 0, "bitlinear: K=%d must be a positive multiple of 128", K);
  HB_REQUIRE(M >= 1 && M <= 4096, "bitlinear: M=%d outside 1..4096", M);
  HB_REQUIRE(d_x != nullptr, "bitlinear: null activation pointer");
  HB_REQUIRE((reinterpret_cast<uintptr_t>(d_x) & 15) == 0, "bitlinear: x must be 16-byte aligned");
  return HB200_OK;
}

}  // namespace hb

using namespace hb;

extern "C" int hb200_bitlinear_forward_multi(hb200_ctx* ctx, const hb200_bitlinear_seg* segs,
                                             int nseg, int K, const float* d_x, int M,
                                             const float* d_rms_gamma, float rms_eps,
                                             float* d_act_scale, hb200_stream stream) {
  int rc = bl_check_common(ctx, K, M, d_x);
  if (rc) return rc;
  HB_REQUIRE(segs && nseg >= 1 && nseg <= kBLMaxSeg, "bitlinear: nseg=%d outside 1..%d", nseg,
             kBLMaxSeg);
  long rows = 0;
  for (int s = 0; s < nseg; ++s) {
    HB_REQUIRE(segs[s].N >= 1, "bitlinear: segment %d has N=%d", s, segs[s].N);
    HB_REQUIRE(segs[s].d_packed && segs[s].d_scale && segs[s].d_y,
               "bitlinear: segment %d has a null weight, scale or output pointer", s);
    HB_REQUIRE((reinterpret_cast<uintptr_t>(segs[s].d_packed) & 15) == 0,
               "bitlinear: segment %d weights must be 16-byte aligned", s);
    rows += segs[s].N;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // tokens per pass over the weights: 128 on the tensor cores, 64 on the dp4a kernel
  const int pass = (K <= 12288 && !ctx->no_mma) ? 128 : 64;
  if (M > pass) {
    for (int m0 = 0; m0 < M; m0 += pass) {
      const int mc = M - m0 < pass ? M - m0 : pass;
      hb200_bitlinear_seg sub[kBLMaxSeg];
      for (int s = 0; s < nseg; ++s) {
        sub[s] = segs[s];
        const size_t o = (size_t)m0 * segs[s].N;
        sub[s].d_y = segs[s].d_y + o;
        if (segs[s].d_residual) sub[s].d_residual = segs[s].d_residual + o;
        if (segs[s].d_acc) sub[s].d_acc = segs[s].d_acc + o;
      }
      rc = hb200_bitlinear_forward_multi(ctx, sub, nseg, K, d_x + (size_t)m0 * K, mc, d_rms_gamma,
                                         rms_eps, d_act_scale ? d_act_scale + m0 : nullptr, stream);
      if (rc) return rc;
    }
    return HB200_OK;
  }
  // 16 or more tokens: a real contraction -> tensor cores (weights still streamed once)
  if (M >= 16 && K <= 12288 && !ctx->no_mma)
    return hb_bitlinear_mma_run(ctx, segs, nseg, K, d_x, M, d_rms_gamma, rms_eps, d_act_scale, st);
  if (M == 1) {  // one token: integer tensor-core matvec when the rows fit shared memory
    rc = hb_bl_mv_run(ctx, segs, nseg, K, 0, d_x, d_rms_gamma, rms_eps, d_act_scale, st);
    if (rc <= 0) return rc;
  }
  const int rt = bl_pick_rt(ctx, rows);
  BLParams p = {};
  int t = 0;
  for (int s = 0; s < nseg; ++s) {
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_packed), segs[s].d_scale,
                segs[s].d_residual, segs[s].d_y, segs[s].d_acc, segs[s].N, t};
    t += (segs[s].N + rt - 1) / rt;
  }
  p.nseg = nseg;
  p.gateup = 0;
  p.ntiles = t;
  p.K = K;
  p.M = M;
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.eps = rms_eps;
  p.act_scale = d_act_scale;
  p.status = ctx->d_status;
  return rt == 4 ? bl_dispatch_wpl<4, false>(ctx, p, st) : bl_dispatch_wpl<2, false>(ctx, p, st);
}

extern "C" int hb200_bitlinear_qkv_rope(hb200_ctx* ctx, const hb200_bitlinear_seg* segs, int K,
                                        const float* d_x, const float* d_rms_gamma, float rms_eps,
                                        const double* d_rope_table, const int32_t* d_pos,
                                        void* d_k_cache, void* d_v_cache, int H, int Hkv, int D,
                                        int cache_slots, int ring, hb200_stream stream) {
  HB_REQUIRE(ctx && segs && d_x && d_rope_table && d_pos && d_k_cache && d_v_cache,
             "bitlinear q/k/v + RoPE: null pointer");
  HB_REQUIRE(H >= 1 && Hkv >= 1 && D >= 2 && D % 2 == 0 && cache_slots >= 1,
             "bitlinear q/k/v + RoPE: H=%d Hkv=%d D=%d slots=%d", H, Hkv, D, cache_slots);
  HB_REQUIRE(segs[0].N == H * D && segs[1].N == Hkv * D && segs[2].N == Hkv * D,
             "bitlinear q/k/v + RoPE: tensors of %d, %d, %d rows for %d/%d heads of %d", segs[0].N,
             segs[1].N, segs[2].N, H, Hkv, D);
  HB_REQUIRE(segs[0].d_y && segs[1].d_y && segs[2].d_y,
             "bitlinear q/k/v + RoPE: q, k and v need f32 output rows (k, v: scratch)");
  int rc = bl_check_common(ctx, K, 1, d_x);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const HbRope rope = {d_rope_table, d_pos, d_k_cache, d_v_cache, D, cache_slots, ring};
  rc = hb_bl_mv_run(ctx, segs, 3, K, 0, d_x, d_rms_gamma, rms_eps, nullptr, st, &rope);
  if (rc <= 0) return rc;
  // a shape the fused kernel does not cover: the two launches it stands for
  rc = hb200_bitlinear_forward_multi(ctx, segs, 3, K, d_x, 1, d_rms_gamma, rms_eps, nullptr, stream);
  if (rc) return rc;
  return hb200_rope_kv_write_angles(ctx, segs[0].d_y, segs[1].d_y, segs[2].d_y, d_k_cache,
                                    d_v_cache, d_pos, d_rope_table, 1, H, Hkv, D, cache_slots,
                                    ring, stream);
}

extern "C" int hb200_bitlinear_forward(hb200_ctx* ctx, const void* d_packed,
                                       const float* d_scale, int K, int N, const float* d_x,
                                       int M, const float* d_rms_gamma, float rms_eps,
                                       const float* d_residual, int32_t* d_acc,
                                       float* d_act_scale, float* d_y, hb200_stream stream) {
  hb200_bitlinear_seg s = {d_packed, d_scale, d_residual, d_y, d_acc, N};
  return hb200_bitlinear_forward_multi(ctx, &s, 1, K, d_x, M, d_rms_gamma, rms_eps, d_act_scale,
                                       stream);
}

extern "C" int hb200_bitlinear_gateup_relu2(hb200_ctx* ctx, const void* d_packed_gate,
                                            const float* d_scale_gate, const void* d_packed_up,
                                            const float* d_scale_up, int K, int N,
                                            const float* d_x, int M, const float* d_rms_gamma,
                                            float rms_eps, float* d_y, hb200_stream stream) {
  int rc = bl_check_common(ctx, K, M, d_x);
  if (rc) return rc;
  HB_REQUIRE(N >= 1, "bitlinear gate/up: N=%d", N);
  HB_REQUIRE(d_packed_gate && d_packed_up && d_scale_gate && d_scale_up && d_y,
             "bitlinear gate/up: null pointer");
  HB_REQUIRE(((reinterpret_cast<uintptr_t>(d_packed_gate) |
               reinterpret_cast<uintptr_t>(d_packed_up)) & 15) == 0,
             "bitlinear gate/up: weights must be 16-byte aligned");
  // tokens per pass: 128 where both products run on the tensor cores into the scratch, else 64
  const int pass = (K <= 12288 && !ctx->no_mma &&
                    kScratchGlu + (size_t)2 * 128 * N * sizeof(float) <= kScratchRowScale)
                       ? 128
                       : 64;
  if (M > pass) {
    for (int m0 = 0; m0 < M; m0 += pass) {
      const int mc = M - m0 < pass ? M - m0 : pass;
      rc = hb200_bitlinear_gateup_relu2(ctx, d_packed_gate, d_scale_gate, d_packed_up, d_scale_up,
                                        K, N, d_x + (size_t)m0 * K, mc, d_rms_gamma, rms_eps,
                                        d_y + (size_t)m0 * N, stream);
      if (rc) return rc;
    }
    return HB200_OK;
  }
  if (M >= 16 && K <= 12288 && !ctx->no_mma &&
      kScratchGlu + (size_t)2 * M * N * sizeof(float) <= kScratchRowScale) {
    // batched: both products on the tensor cores into scratch (the region may run into the
    // staging area of the 16-bit products, which no ternary operator uses), then the GLU
    ScratchUse use(ctx, static_cast<cudaStream_t>(stream));
    float* g = reinterpret_cast<float*>(static_cast<uint8_t*>(ctx->d_scratch) + kScratchGlu);
    float* u = g + (size_t)M * N;
    hb200_bitlinear_seg segs[2] = {{d_packed_gate, d_scale_gate, nullptr, g, nullptr, N},
                                   {d_packed_up, d_scale_up, nullptr, u, nullptr, N}};
    rc = hb_bitlinear_mma_run(ctx, segs, 2, K, d_x, M, d_rms_gamma, rms_eps, nullptr,
                              static_cast<cudaStream_t>(stream));
    if (rc) return rc;
    return hb200_relu2_mul(ctx, g, u, (long)M * N, d_y, stream);
  }
  if (M == 1) {
    const hb200_bitlinear_seg gs[2] = {{d_packed_gate, d_scale_gate, nullptr, d_y, nullptr, N},
                                       {d_packed_up, d_scale_up, nullptr, d_y, nullptr, N}};
    rc = hb_bl_mv_run(ctx, gs, 2, K, 1, d_x, d_rms_gamma, rms_eps, nullptr,
                      static_cast<cudaStream_t>(stream));
    if (rc <= 0) return rc;
  }
  // a gate/up tile streams 2*RT rows, so the row count that matters doubles
  const int rt = bl_pick_rt(ctx, 2L * N) == 4 ? 4 : 2;
  BLParams p = {};
  p.seg[0] = {static_cast<const uint8_t*>(d_packed_gate), d_scale_gate, nullptr, d_y, nullptr, N, 0};
  p.seg[1] = {static_cast<const uint8_t*>(d_packed_up), d_scale_up, nullptr, d_y, nullptr, N, 0};
  p.nseg = 2;
  p.gateup = 1;
  p.ntiles = (N + rt - 1) / rt;
  p.K = K;
  p.M = M;
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.eps = rms_eps;
  p.act_scale = nullptr;
  p.status = ctx->d_status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return rt == 4 ? bl_dispatch_wpl<4, true>(ctx, p, st) : bl_dispatch_wpl<2, true>(ctx, p, st);
}
