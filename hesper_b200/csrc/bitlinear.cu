// bitlinear.cu -- ternary (i2_s) x int8 matvec for sm_100a.
//
// What it computes is BitLinearSpec.forward (Hesper/Layers/BitLinearSpec.lean:65-91)
// on int8 activations: acc[n] = sum_k t[n,k]*q[k] exactly in int32, then
// y = ((float)acc*d)*s (+residual).  The reference's kernels for the same layer
// are fusedBitLinearM1Kernel and its residual / RMSNorm / gate-up variants
// (Hesper/Layers/BitLinear.lean:297,361,447,553).
//
// How it runs on B200:
//   * rows are split evenly over the grid (one CTA per SM) and then over the
//     warps of a CTA; every warp is its own streaming engine: lane 0 pulls the
//     warp's rows global->shared with 1-D TMA bulk copies completed on a per-warp
//     mbarrier ring, so no CTA-wide barrier sits in the streaming loop;
//   * the weight prefetch is issued BEFORE griddepcontrol.wait: under programmatic
//     dependent launch the bytes of this layer are in flight while the previous
//     kernel of the decode step is still finishing;
//   * meanwhile the whole CTA runs the activation prologue (optional RMSNorm,
//     absmax, int8 quantisation) into shared memory, laid out so that the four
//     2-bit planes of a packed word meet their activations as four dp4a operands;
//   * unpacking is four ANDs per 16 weights: plane p of word w is w & (3 << 2p)
//     per byte, i.e. the code scaled by 4^p, which dp4a.u32.s32 multiplies
//     directly; the scale is shifted out once per row and sum(q) is subtracted
//     once (value = code - 1);
//   * a transposing shuffle reduction turns 8 per-lane row partials into 8 row
//     sums with 9 shuffles.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace hb {

constexpr int kBLMaxSeg = 4;
constexpr int kBLRowsPerTile = 8;  // accumulator slots per warp tile

struct BLSeg {
  const uint8_t* w;
  const float* scale;
  const float* residual;
  float* y;
  int32_t* acc;
  int N;
  int vrow0;  // first virtual row of this segment
};

struct BLParams {
  BLSeg seg[kBLMaxSeg];
  int nseg;
  int gateup;      // 1: seg[0] = gate, seg[1] = up, fused ReLU^2 GLU epilogue
  int vrows;       // total virtual rows (sum of N; N for gate/up)
  int K;
  int M;           // tokens
  int rt;          // rows per tile actually used (<= 8; <= 4 for gate/up)
  int stages;      // ring depth per warp
  int stage_rows;  // row slots per stage in shared memory (rt, or 2*rt for gate/up)
  const float* x;  // [M][K]
  const float* gamma;
  float eps;
  float* act_scale;  // nullable [M]
  uint32_t* status;
};

// Block-wide reductions over `nwarps` warps through a small shared scratch.
__device__ __forceinline__ float block_max(float v, float* scratch, int warp, int lane,
                                           int nwarps) {
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int i = 1; i < nwarps; ++i) r = fmaxf(r, scratch[i]);
  return r;
}
__device__ __forceinline__ double block_sum_f64(double v, double* scratch, int warp, int lane,
                                                int nwarps) {
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double r = 0.0;
  for (int i = 0; i < nwarps; ++i) r += scratch[i];
  return r;
}
__device__ __forceinline__ int block_sum_i32(int v, int* scratch, int warp, int lane,
                                             int nwarps) {
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  int r = 0;
  for (int i = 0; i < nwarps; ++i) r += scratch[i];
  return r;
}

// Sum of 8 per-lane partials across the warp: afterwards every lane holds the
// full sum of slot (lane >> 2).
__device__ __forceinline__ int transpose_reduce8(const int (&a)[8], int lane) {
  int v4[4], v2[2], v1;
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int send = b4 ? a[i] : a[i + 4];
    int keep = b4 ? a[i + 4] : a[i];
    v4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int send = b3 ? v4[i] : v4[i + 2];
    int keep = b3 ? v4[i + 2] : v4[i];
    v2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  {
    int send = b2 ? v2[0] : v2[1];
    int keep = b2 ? v2[1] : v2[0];
    v1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
  v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
  return v1;
}

// Which segment holds virtual row v, and how many rows may one tile take from v
// without crossing the segment end, the warp's range end or the tile size.
__device__ __forceinline__ void bl_tile_at(const BLParams& p, int v, int vend, int& seg,
                                           int& row, int& nr) {
  seg = 0;
  if (!p.gateup) {
#pragma unroll
    for (int s = 1; s < kBLMaxSeg; ++s)
      if (s < p.nseg && v >= p.seg[s].vrow0) seg = s;
  }
  row = v - p.seg[seg].vrow0;
  int lim = p.seg[seg].N - row;
  nr = min(p.rt, min(lim, vend - v));
}

template <int WPL, int MT>
__global__ void __launch_bounds__(MT == 1 ? 512 : 256, 1)
    bitlinear_kernel(const __grid_constant__ BLParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int K = p.K;
  const int words = K >> 4;     // packed u32 per row
  const int rowbytes = K >> 2;  // packed bytes per row
  const int S = p.stages;
  const int stage_bytes = p.stage_rows * rowbytes;

  // shared memory carve-up (bl_smem_bytes on the host mirrors it)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [nwarps][S]
  size_t off = (size_t)nwarps * S * sizeof(uint64_t);
  off = (off + 127) & ~size_t(127);
  double* red_f64 = reinterpret_cast<double*>(smem + off);
  off += 32 * sizeof(double);
  float* red_f32 = reinterpret_cast<float*>(smem + off);
  off += 32 * sizeof(float);
  int* red_i32 = reinterpret_cast<int*>(smem + off);
  off += 32 * sizeof(int);
  float* tok_d = reinterpret_cast<float*>(smem + off);  // [MT] activation scales
  off += 8 * sizeof(float);
  int* tok_sumq = reinterpret_cast<int*>(smem + off);  // [MT] sum of int8 activations
  off += 8 * sizeof(int);
  off = (off + 127) & ~size_t(127);
  float* xf = reinterpret_cast<float*>(smem + off);  // [K] staging of one token
  off += (size_t)K * sizeof(float);
  uint32_t* xq = reinterpret_cast<uint32_t*>(smem + off);  // [MT][4 planes][words]
  off += (size_t)MT * K;
  off = (off + 127) & ~size_t(127);
  uint8_t* wstage = smem + off + (size_t)warp * S * stage_bytes;
  uint64_t* mybar = bars + warp * S;

  // this warp's virtual-row range: rows split evenly over CTAs, then over warps
  const int G = gridDim.x;
  const int c0 = (int)(((long long)blockIdx.x * p.vrows) / G);
  const int c1 = (int)(((long long)(blockIdx.x + 1) * p.vrows) / G);
  const int crow = c1 - c0;
  const int v0 = c0 + (int)(((long long)warp * crow) / nwarps);
  const int v1 = c0 + (int)(((long long)(warp + 1) * crow) / nwarps);

  if (lane == 0) {
    for (int s = 0; s < S; ++s) mbar_init(&mybar[s], 1);
    fence_mbar_init();
  }
  __syncwarp();
  const uint64_t pol = policy_evict_first();

  // Ring bookkeeping is warp-uniform: every lane tracks the cursors, lane 0 issues.
  // Tile number t (counted over all passes) lives in stage t % S and completes
  // phase (t / S) & 1 of that stage's mbarrier.
  int issued = 0, consumed = 0, vprod = v0;
  auto produce = [&]() {
    int seg, row, nr;
    bl_tile_at(p, vprod, v1, seg, row, nr);
    if (lane == 0) {
      const int stage = issued % S;
      uint8_t* dst = wstage + (size_t)stage * stage_bytes;
      const uint32_t bytes = (uint32_t)nr * rowbytes;
      if (!p.gateup) {
        mbar_arrive_expect_tx(&mybar[stage], bytes);
        bulk_g2s_stream(dst, p.seg[seg].w + (size_t)row * rowbytes, bytes, &mybar[stage], pol);
      } else {
        mbar_arrive_expect_tx(&mybar[stage], 2 * bytes);
        bulk_g2s_stream(dst, p.seg[0].w + (size_t)row * rowbytes, bytes, &mybar[stage], pol);
        bulk_g2s_stream(dst + (size_t)p.rt * rowbytes, p.seg[1].w + (size_t)row * rowbytes,
                        bytes, &mybar[stage], pol);
      }
    }
    vprod += nr;
    ++issued;
  };

  // ---- weight prefetch: independent of the previous kernel ------------------
  while (issued < S && vprod < v1) produce();
  pdl_trigger();
  pdl_wait();  // activations (and residuals) come from the previous kernel

  const int nchunks = (words + 32 * WPL - 1) / (32 * WPL);

  for (int m0 = 0; m0 < p.M; m0 += MT) {
    // ---- activation prologue: RMSNorm (optional), absmax, int8 --------------
    if (m0 > 0) __syncthreads();  // all warps are done with the previous xq
    for (int mt = 0; mt < MT; ++mt) {
      const int m = m0 + mt;
      uint32_t* xqm = xq + (size_t)mt * (K >> 2);
      if (m >= p.M) {  // padding token: zeros
        for (int i = tid; i < (K >> 2); i += blockDim.x) xqm[i] = 0u;
        if (tid == 0) {
          tok_d[mt] = 0.f;
          tok_sumq[mt] = 0;
        }
        continue;
      }
      const float4* xg = reinterpret_cast<const float4*>(p.x + (size_t)m * K);
      float4* xs = reinterpret_cast<float4*>(xf);
      float amax = 0.f;
      if (p.gamma) {
        double ss = 0.0;
        for (int i = tid; i < (K >> 2); i += blockDim.x) {
          float4 v = __ldg(xg + i);
          xs[i] = v;
          ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
        }
        ss = block_sum_f64(ss, red_f64, warp, lane, nwarps);
        const float rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
        const float4* gg = reinterpret_cast<const float4*>(p.gamma);
        for (int i = tid; i < (K >> 2); i += blockDim.x) {
          float4 v = xs[i], g = __ldg(gg + i);
          v.x = __fmul_rn(__fmul_rn(v.x, rinv), g.x);
          v.y = __fmul_rn(__fmul_rn(v.y, rinv), g.y);
          v.z = __fmul_rn(__fmul_rn(v.z, rinv), g.z);
          v.w = __fmul_rn(__fmul_rn(v.w, rinv), g.w);
          xs[i] = v;
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
      } else {
        for (int i = tid; i < (K >> 2); i += blockDim.x) {
          float4 v = __ldg(xg + i);
          xs[i] = v;
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
      }
      amax = block_max(amax, red_f32, warp, lane, nwarps);
      const float d = __fdiv_rn(amax, 127.0f);
      int sumq = 0;
      for (int i = tid; i < (K >> 2); i += blockDim.x) {
        float4 v = xs[i];
        int q0 = 0, q1 = 0, q2 = 0, q3 = 0;
        if (d != 0.f) {
          q0 = __float2int_rn(__fdiv_rn(v.x, d));
          q1 = __float2int_rn(__fdiv_rn(v.y, d));
          q2 = __float2int_rn(__fdiv_rn(v.z, d));
          q3 = __float2int_rn(__fdiv_rn(v.w, d));
        }
        sumq += q0 + q1 + q2 + q3;
        // elements k = 4i..4i+3 sit in group g, plane s, byte-quad wi of the group
        const int k = i << 2;
        const int g = k >> 7, c = k & 127, s = c >> 5, wi = (c & 31) >> 2;
        const uint32_t pk = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) |
                            ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)(q3 & 0xff) << 24);
        xqm[s * words + g * 8 + wi] = pk;
      }
      sumq = block_sum_i32(sumq, red_i32, warp, lane, nwarps);
      if (tid == 0) {
        tok_d[mt] = d;
        tok_sumq[mt] = sumq;
        if (p.act_scale && blockIdx.x == 0) p.act_scale[m] = d;
      }
    }
    __syncthreads();

    // ---- streaming main loop (per warp) --------------------------------------
    // Token groups after the first stream the weights again (from L2 by then).
    if (m0 > 0) {
      vprod = v0;
      for (int n = 0; n < S && vprod < v1; ++n) produce();
    }
    int vcons = v0;
    while (vcons < v1) {
      const int stage = consumed % S;
      const uint32_t parity = (uint32_t)((consumed / S) & 1);
      int seg, row, nr;
      bl_tile_at(p, vcons, v1, seg, row, nr);
      mbar_wait(&mybar[stage], parity, p.status);
      const uint32_t* ws = reinterpret_cast<const uint32_t*>(wstage + (size_t)stage * stage_bytes);

      int acc[MT][kBLRowsPerTile];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < kBLRowsPerTile; ++r) acc[mt][r] = 0;

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
            const uint32_t* xqm = xq + (size_t)mt * (K >> 2);
#pragma unroll
            for (int s = 0; s < 4; ++s) xr[mt][i][s] = ok ? xqm[s * words + j] : 0u;
          }
        }
#pragma unroll
        for (int r = 0; r < kBLRowsPerTile; ++r) {
          // accumulator slot r -> row of the stage: plain tiles use slots 0..nr-1;
          // gate/up tiles keep gate rows in slots 0..3 and up rows in slots 4..7
          const bool live = p.gateup ? ((r & 3) < nr) : (r < nr);
          if (live) {
            const int srow = p.gateup ? ((r < 4) ? r : (p.rt + r - 4)) : r;
            const uint32_t* wr = ws + srow * words;
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
      }
      __syncwarp();  // every lane has finished reading this stage
      if (vprod < v1) produce();  // refill it with the tile S ahead

      // ---- reduce and store ---------------------------------------------------
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = m0 + mt;
        const int total = transpose_reduce8(acc[mt], lane) - tok_sumq[mt];
        const int slot = lane >> 2;
        if (!p.gateup) {
          if ((lane & 3) == 0 && slot < nr && m < p.M) {
            const BLSeg& sg = p.seg[seg];
            const size_t o = (size_t)m * sg.N + row + slot;
            if (sg.acc) sg.acc[o] = total;
            float v = __fmul_rn(__fmul_rn((float)total, tok_d[mt]), __ldg(sg.scale));
            if (sg.residual) v = __fadd_rn(v, sg.residual[o]);
            sg.y[o] = v;
          }
        } else {
          const int up = __shfl_down_sync(0xffffffffu, total, 16);
          if ((lane & 3) == 0 && slot < 4 && slot < nr && m < p.M) {
            const size_t o = (size_t)m * p.seg[0].N + row + slot;
            const float g = __fmul_rn(__fmul_rn((float)total, tok_d[mt]), __ldg(p.seg[0].scale));
            const float u = __fmul_rn(__fmul_rn((float)up, tok_d[mt]), __ldg(p.seg[1].scale));
            const float r = g > 0.f ? g : 0.f;
            p.seg[0].y[o] = __fmul_rn(__fmul_rn(r, r), u);
          }
        }
      }
      vcons += nr;
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

template <int WPL, int MT>
static cudaError_t bl_launch(const BLParams& p, int grid, int threads, size_t smem,
                             cudaStream_t st, bool pdl) {
  auto kern = bitlinear_kernel<WPL, MT>;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    configured = smem;
  }
  return launch_pdl(kern, dim3(grid), dim3(threads), smem, st, pdl, p);
}

// Shared memory of one CTA; mirrors the carve-up at the top of the kernel.
static size_t bl_smem_bytes(int nwarps, int stages, int stage_rows, int K, int MT) {
  auto up128 = [](size_t v) { return (v + 127) & ~size_t(127); };
  size_t off = up128((size_t)nwarps * stages * 8);
  off += 32 * 8 + 32 * 4 + 32 * 4 + 8 * 4 + 8 * 4;
  off = up128(off);
  off += (size_t)K * 4 + (size_t)MT * K;
  off = up128(off);
  return off + (size_t)nwarps * stages * stage_rows * (size_t)(K / 4);
}

static int bl_run(hb200_ctx* ctx, BLParams& p, cudaStream_t st) {
  const int K = p.K;
  const int words = K / 16;
  const int MT = p.M == 1 ? 1 : 4;
  const int threads = MT == 1 ? 512 : 256;
  const int nwarps = threads / 32;
  const int wpl = pick_wpl(words);
  const int grid = p.vrows < ctx->sm_count ? p.vrows : ctx->sm_count;

  // Tile height and ring depth: take the warp's whole row range in one tile when
  // it fits (everything in flight at once), else the deepest ring that fits.
  const int max_rt = p.gateup ? 4 : 8;
  const int rows_per_cta = (p.vrows + grid - 1) / grid;
  const int rows_per_warp = (rows_per_cta + nwarps - 1) / nwarps;
  const size_t budget = (size_t)ctx->smem_optin;
  int rt = rows_per_warp < max_rt ? rows_per_warp : max_rt;
  if (rt < 1) rt = 1;
  int stages = 0;
  size_t smem = 0;
  for (;;) {
    const int tiles = (rows_per_warp + rt - 1) / rt;
    const int srows = p.gateup ? 2 * rt : rt;
    const int smin = tiles > 1 ? 2 : 1;
    for (int s = (tiles < 4 ? tiles : 4); s >= smin; --s) {
      const size_t total = bl_smem_bytes(nwarps, s, srows, K, MT);
      if (total <= budget) {
        stages = s;
        smem = total;
        break;
      }
    }
    if (stages) break;
    if (rt == 1) {
      set_error("bitlinear: K=%d does not fit the shared-memory budget", K);
      return HB200_ERR_UNSUPPORTED;
    }
    rt = rt / 2;
  }
  p.rt = rt;
  p.stages = stages;
  p.stage_rows = p.gateup ? 2 * rt : rt;
  p.status = ctx->d_status;

  cudaError_t e;
#define HB_BL_CASE(W)                                                      \
  case W:                                                                  \
    e = (MT == 1) ? bl_launch<W, 1>(p, grid, threads, smem, st, ctx->pdl)  \
                  : bl_launch<W, 4>(p, grid, threads, smem, st, ctx->pdl); \
    break;
  switch (wpl) {
    HB_BL_CASE(4)
    HB_BL_CASE(5)
    HB_BL_CASE(6)
    HB_BL_CASE(7)
    HB_BL_CASE(8)
    default:
      set_error("bitlinear: internal: no kernel for %d words per lane", wpl);
      return HB200_ERR_UNSUPPORTED;
  }
#undef HB_BL_CASE
  if (e != cudaSuccess) return cuda_fail(e, "bitlinear launch");
  return HB200_OK;
}

static int bl_check_common(hb200_ctx* ctx, int K, int M, const float* d_x) {
  HB_REQUIRE(ctx != nullptr, "bitlinear: null context");
  HB_REQUIRE(K > 0 && K % 128 == 0, "bitlinear: K=%d must be a positive multiple of 128", K);
  HB_REQUIRE(M >= 1 && M <= 64, "bitlinear: M=%d outside 1..64", M);
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
  BLParams p = {};
  int v = 0;
  for (int s = 0; s < nseg; ++s) {
    HB_REQUIRE(segs[s].N >= 1, "bitlinear: segment %d has N=%d", s, segs[s].N);
    HB_REQUIRE(segs[s].d_packed && segs[s].d_scale && segs[s].d_y,
               "bitlinear: segment %d has a null weight, scale or output pointer", s);
    HB_REQUIRE((reinterpret_cast<uintptr_t>(segs[s].d_packed) & 15) == 0,
               "bitlinear: segment %d weights must be 16-byte aligned", s);
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_packed), segs[s].d_scale,
                segs[s].d_residual, segs[s].d_y, segs[s].d_acc, segs[s].N, v};
    v += segs[s].N;
  }
  p.nseg = nseg;
  p.gateup = 0;
  p.vrows = v;
  p.K = K;
  p.M = M;
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.eps = rms_eps;
  p.act_scale = d_act_scale;
  return bl_run(ctx, p, static_cast<cudaStream_t>(stream));
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
  HB_REQUIRE(((reinterpret_cast<uintptr_t>(d_packed_gate) | reinterpret_cast<uintptr_t>(d_packed_up)) & 15) == 0,
             "bitlinear gate/up: weights must be 16-byte aligned");
  BLParams p = {};
  p.seg[0] = {static_cast<const uint8_t*>(d_packed_gate), d_scale_gate, nullptr, d_y, nullptr, N, 0};
  p.seg[1] = {static_cast<const uint8_t*>(d_packed_up), d_scale_up, nullptr, d_y, nullptr, N, 0};
  p.nseg = 2;
  p.gateup = 1;
  p.vrows = N;
  p.K = K;
  p.M = M;
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.eps = rms_eps;
  p.act_scale = nullptr;
  return bl_run(ctx, p, static_cast<cudaStream_t>(stream));
}
