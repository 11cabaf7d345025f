// kquant.cu -- GGUF Q4_K / Q8_0 dequant-fused matvec for sm_100a, f32 activations.
//
// What it computes: y[n] = sum_k dequant(W)[n,k] * x[k] with the block formats of
// Hesper/Quantization/Q4_K_M.lean:13-52,120-144 (Q4_K: w = d*sc*q - dmin*m) and
// Hesper/Layers/Linear.lean:6187-6223 (Q8_0: w = d*q).  The reference's kernels
// for the same layers are mulMvQ4KF32Kernel (Hesper/WGSL/MulMvQ4K.lean:46), the
// dp4a family (Hesper/Layers/Linear.lean:1777-3450) and fusedQ8_0LinearKernel
// (:6192); the fused gate/up GELU epilogue follows Hesper/Layers/FusedFFNSpec.lean:42-122.
//
// How it runs on B200:
//   * same streaming skeleton as the ternary kernel: rows are cut into tiles of
//     RT rows, tiles are split evenly over the grid and dealt round-robin to the
//     warps; each warp pulls its tiles global->shared with 1-D TMA bulk copies on
//     its own mbarrier ring, issued before griddepcontrol.wait so the weights of
//     this layer fly while the previous kernel finishes;
//   * the integer pipe does the dot products: activations are block-quantised per
//     32 elements to 16 bits (x ~ dx * (256*hi + lo), hi int8, lo uint8), which is
//     finer than f16 and keeps the result within 1e-4 of an f64 evaluation, while a
//     4-bit quant needs only one AND per 4 weights (the high nibble is used in
//     place, its factor 16 folded into the activation scale) and two dp4a;
//   * the work unit of a lane is one 64-weight chunk (a Q4_K sub-block pair or two
//     Q8_0 blocks): lane l owns chunk l of the row for every row of the tile, so
//     its 32 activation registers are loaded once per tile; the six-bit scales of
//     a Q4_K chunk are decoded four at a time with mask arithmetic on the packed
//     words; the min term uses exact f32 sub-block sums of x;
//   * per-lane row partials are summed with a transposing shuffle reduction.
#include "common.cuh"

namespace hb {


constexpr int kKQMaxSeg = 4;
constexpr int kKQBatchedFrom = 16;  // tokens from which the tensor-core path takes over
constexpr int kKQThreads = 384;
constexpr int kKQWarps = kKQThreads / 32;

struct KQSeg {
  const uint8_t* w;
  const float* residual;
  float* y;
  int N;
  int tile0;
};

struct KQParams {
  KQSeg seg[kKQMaxSeg];
  int nseg;
  int ntiles;
  int K;
  int M;
  int stages;   // tiles a warp keeps in flight
  int nslots;   // stage slots of the CTA: min(warps*stages, most tiles any CTA owns)
  const float* x;
  const float* gamma;
  float eps;
  uint32_t* status;
  // optional step in front of the prologue: x' = pre_base + rmsnorm(x) * pre_gamma, which the
  // matvec (and its own optional RMSNorm) then consumes; CTA 0 also writes x' to pre_out
  const float* pre_base;
  const float* pre_gamma;
  float* pre_out;
};

template <int NS>
__device__ __forceinline__ float transpose_reduce_f(const float (&a)[NS], int lane) {
  float v[NS];
#pragma unroll
  for (int i = 0; i < NS; ++i) v[i] = a[i];
  int bit = 16;
#pragma unroll
  for (int n = NS; n > 1; n >>= 1) {
    const bool hi = lane & bit;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = hi ? v[i] : v[i + n / 2];
      const float keep = hi ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
    }
    bit >>= 1;
  }
#pragma unroll
  for (; bit >= 1; bit >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], bit);
  return v[0];
}

// The two low bytes of v as floats (I2F with a byte selector, no masking).
__device__ __forceinline__ void u8x2_to_f(uint32_t v, float& a, float& b) {
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
      "mov.b32 {t0, t1, t2, t3}, %2;\n\t"
      "cvt.rn.f32.u8 %0, t0;\n\t"
      "cvt.rn.f32.u8 %1, t1;\n\t}"
      : "=f"(a), "=f"(b)
      : "r"(v));
}

// Lane-constant selectors for the 6-bit scale / min pair of chunk c (sub-blocks 2c, 2c+1)
// out of the 12 packed bytes w0..w2 (Hesper/Quantization/Q4_K_M.lean:120-144):
//   c < 2 : sc = (w0 >> sh) & 0x3F3F                         m = (w1 >> sh) & 0x3F3F
//   c >= 2: sc = ((w2 >> sh) & 0x0F0F) | ((w0 >> sh+2) & 0x3030)
//           m  = ((w2 >> sh+4) & 0x0F0F) | ((w1 >> sh+2) & 0x3030)      with sh = 16*(c&1)
// Written with masks and shift counts that depend only on c, so every lane runs the same
// instructions whatever its chunk.
struct Q4KSel {
  uint32_t sh, mask_lo, mask_hi, m_extra;  // m_extra: extra right shift of w2 for the mins
  bool upper;                              // c >= 2
};
__device__ __forceinline__ Q4KSel q4k_sel(int c) {
  Q4KSel s;
  s.upper = c >= 2;
  s.sh = (uint32_t)(c & 1) * 16u;
  s.mask_lo = s.upper ? 0x0F0Fu : 0x3F3Fu;
  s.mask_hi = s.upper ? 0x3030u : 0u;
  s.m_extra = s.upper ? 4u : 0u;
  return s;
}

// One 64-weight Q4_K chunk (sub-blocks 2c and 2c+1 of a super-block) against its
// 64 activations.  blk = super-block base in shared memory; xh/xl = the 16+16
// words of the hi/lo activation planes of the chunk; tab = {dx_lo, dx_hi/16,
// sumx_lo, sumx_hi} of the two sub-blocks.
__device__ __forceinline__ float q4k_chunk(const uint8_t* blk, int c, const Q4KSel& sel,
                                           const uint32_t (&xh)[16], const uint32_t (&xl)[16],
                                           float4 tab) {
  const uint4 hdr = *reinterpret_cast<const uint4*>(blk);  // d|dmin, scales[0..11]
  const uint4 qa = *reinterpret_cast<const uint4*>(blk + 16 + 32 * c);
  const uint4 qb = *reinterpret_cast<const uint4*>(blk + 32 + 32 * c);
  const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
  int lh = 0, ll = 0, hh = 0, hl = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t lo = q[i] & 0x0F0F0F0Fu, hi = q[i] & 0xF0F0F0F0u;
    lh = dp4a_us(lo, xh[i], lh);
    ll = dp4a_uu(lo, xl[i], ll);
    hh = dp4a_us(hi, xh[8 + i], hh);
    hl = dp4a_uu(hi, xl[8 + i], hl);
  }
  const float fL = (float)(lh * 256 + ll);
  const float fH = (float)(hh * 256 + hl);  // carries the factor 16 of the high nibble
  const uint32_t wa = sel.upper ? hdr.w : hdr.y;   // low bits of the scales
  const uint32_t wm = sel.upper ? hdr.w : hdr.z;   // low bits of the mins
  const uint32_t sc2 = ((wa >> sel.sh) & sel.mask_lo) | ((hdr.y >> (sel.sh + 2)) & sel.mask_hi);
  const uint32_t m2 =
      ((wm >> (sel.sh + sel.m_extra)) & sel.mask_lo) | ((hdr.z >> (sel.sh + 2)) & sel.mask_hi);
  float scl, sch, ml, mh;
  u8x2_to_f(sc2, scl, sch);
  u8x2_to_f(m2, ml, mh);
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));
  const float main = fmaf(sch * tab.y, fH, (scl * tab.x) * fL);
  const float mins = fmaf(mh, tab.w, ml * tab.z);
  return fmaf(dd.x, main, -(dd.y * mins));
}

// Two consecutive Q8_0 blocks (68 bytes, 4-byte aligned) against 64 activations.
// The first block's quants start 2 bytes into a word and are realigned with
// funnel shifts; the second block's are word aligned.
__device__ __forceinline__ float q80_pair(const uint8_t* pair, const uint32_t (&xh)[16],
                                          const uint32_t (&xl)[16], float4 tab) {
  const uint32_t* W = reinterpret_cast<const uint32_t*>(pair);
  uint32_t w[17];
#pragma unroll
  for (int i = 0; i < 17; ++i) w[i] = W[i];
  int ah = 0, al = 0, bh = 0, bl = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t q0 = __funnelshift_r(w[i], w[i + 1], 16);
    const uint32_t q1 = w[9 + i];
    ah = dp4a_ss(q0, xh[i], ah);
    al = dp4a_su(q0, xl[i], al);
    bh = dp4a_ss(q1, xh[8 + i], bh);
    bl = dp4a_su(q1, xl[8 + i], bl);
  }
  const float d0 = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xffffu)));
  const float d1 = __half2float(__ushort_as_half((unsigned short)(w[8] >> 16)));
  return d0 * tab.x * (float)(ah * 256 + al) + d1 * tab.y * (float)(bh * 256 + bl);
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
  // 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715 x^3))), Hesper/Layers/FusedFFNSpec.lean:42-45
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}

// FMT: 12 = Q4_K, 8 = Q8_0 (GGUF type ids).  RT rows per tile (a gate/up tile
// holds RT gate rows and RT up rows).  GU: fused gelu_tanh(gate)*up.
template <int FMT, int RT, bool GU>
__global__ void __launch_bounds__(kKQThreads, 1) kquant_kernel(const __grid_constant__ KQParams p) {
  constexpr int kRows = GU ? 2 * RT : RT;      // rows held by one stage
  constexpr int kNS = kRows <= 2 ? 2 : (kRows <= 4 ? 4 : 8);  // reduction width
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K;
  const int nchunk = K >> 6;  // 64-weight chunks per row
  const int rowbytes = FMT == 12 ? (K >> 8) * 144 : (K >> 5) * 34;
  const int S = p.stages;
  const int stage_bytes = kRows * rowbytes;

  // shared memory carve-up (kq_smem_bytes mirrors it)
  // Stage slots are interleaved over the warps: the warp's k-th tile sits in slot
  // warp + (k % S) * warps.  When every tile of the CTA is resident at once this makes the
  // slot simply the tile's index in the CTA, so no slot is wasted on a warp with fewer tiles.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);  // [nslots]
  size_t off = ((size_t)p.nslots * sizeof(uint64_t) + 127) & ~size_t(127);
  double* red_f64 = reinterpret_cast<double*>(smem + off);  // [32]: two sets of warp sums
  off += 32 * sizeof(double);
  uint32_t* xhi = reinterpret_cast<uint32_t*>(smem + off);  // [K] int8 hi plane
  off += (size_t)K;
  uint32_t* xlo = reinterpret_cast<uint32_t*>(smem + off);  // [K] uint8 lo plane
  off += (size_t)K;
  float4* xtab = reinterpret_cast<float4*>(smem + off);  // [K/64] chunk scales and sums
  off += (size_t)nchunk * sizeof(float4);
  float4* xs4 = reinterpret_cast<float4*>(smem + off);  // [K] floats, only with the pre-step
  if (p.pre_gamma) off += (size_t)K * sizeof(float);
  off = (off + 127) & ~size_t(127);
  uint8_t* wstage = smem + off;
  auto slot_of = [&](int k) { return warp + (k % S) * kKQWarps; };

  const int G = gridDim.x;
  const int t0 = (int)(((long long)blockIdx.x * p.ntiles) / G);
  const int t1 = (int)(((long long)(blockIdx.x + 1) * p.ntiles) / G);

  if (lane == 0) {
    for (int s = 0; s < S; ++s)
      if (slot_of(s) < p.nslots) mbar_init(&bars[slot_of(s)], 1);
    fence_mbar_init();
  }
  if (tid < 32) red_f64[tid] = 0.0;
  __syncwarp();
  const uint64_t pol = policy_evict_first();

  auto tile_at = [&](int t, int& seg, int& row, int& nr) {
    seg = 0;
    if (!GU) {
#pragma unroll
      for (int s = 1; s < kKQMaxSeg; ++s)
        if (s < p.nseg && t >= p.seg[s].tile0) seg = s;
    }
    row = (t - p.seg[seg].tile0) * RT;
    nr = min(RT, p.seg[seg].N - row);
  };

  int issued = 0, consumed = 0, tprod = t0 + warp;
  auto produce = [&]() {
    int seg, row, nr;
    tile_at(tprod, seg, row, nr);
    if (lane == 0) {
      const int slot = slot_of(issued);
      uint8_t* dst = wstage + (size_t)slot * stage_bytes;
      const uint32_t bytes = (uint32_t)nr * rowbytes;
      if (!GU) {
        mbar_arrive_expect_tx(&bars[slot], bytes);
        bulk_g2s_stream(dst, p.seg[seg].w + (size_t)row * rowbytes, bytes, &bars[slot], pol);
      } else {
        mbar_arrive_expect_tx(&bars[slot], 2 * bytes);
        bulk_g2s_stream(dst, p.seg[0].w + (size_t)row * rowbytes, bytes, &bars[slot], pol);
        bulk_g2s_stream(dst + (size_t)RT * rowbytes, p.seg[1].w + (size_t)row * rowbytes, bytes,
                        &bars[slot], pol);
      }
    }
    tprod += kKQWarps;
    ++issued;
  };

  // ---- weight prefetch, independent of the previous kernel --------------------
  while (issued < S && tprod < t1) produce();
  const int M = p.M;
  const float* const xbase = p.x;
  const float* const gamma = p.gamma;
  // Rows of up to 2 float4 per thread are kept in registers from their first read to the
  // quantisation; the norm weights are constants of the model and are fetched here, before
  // the wait on the previous kernel.
  constexpr int kHeld = 2;
  const int nvec = K >> 2;
  const bool held = nvec <= kHeld * kKQThreads;
  float4 hgm[kHeld];
#pragma unroll
  for (int j = 0; j < kHeld; ++j) {
    const int i = tid + j * kKQThreads;
    hgm[j] = (held && gamma && i < nvec) ? __ldg(reinterpret_cast<const float4*>(gamma) + i)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_trigger();
  pdl_wait();

  const Q4KSel sel_main = q4k_sel(lane & 3);  // in whole passes a lane's chunk index is lane & 3
  const int npass = nchunk >> 5;   // whole passes: lane l owns chunk pass*32 + l
  const int rem = nchunk & 31;     // chunks left per row; rem*kRows tasks per tile
  const int nrem_iter = (rem * kRows + 31) >> 5;
  const uint32_t rem_magic = rem ? 0xFFFFFFFFu / (uint32_t)rem + 1u : 0u;  // idx / rem by multiply

  for (int m = 0; m < M; ++m) {
    // ---- activation prologue: (RMSNorm), per-32 block 16-bit quantisation ------
    __syncthreads();
    const float4* xg = reinterpret_cast<const float4*>(xbase + (size_t)m * K);
    const bool pre = p.pre_gamma != nullptr;
    float rinv = 1.f;
    double ss2 = 0.0;  // sum of squares of the row the matvec consumes, when already known
    float4 hx[kHeld];  // that row, when held in registers
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const int i = tid + j * kKQThreads;
      hx[j] = (held && !pre && i < nvec) ? __ldcg(xg + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (pre) {
      // x' = base + rmsnorm(x) * pre_gamma, same operation order as the standalone kernel.
      // Rows of up to 2 float4 per thread stay in registers with their gamma and base, so
      // that all loads of the step are in flight together (one memory round trip).
      const float4* pg = reinterpret_cast<const float4*>(p.pre_gamma);
      const float4* bg = reinterpret_cast<const float4*>(p.pre_base + (size_t)m * K);
      float4* og = reinterpret_cast<float4*>(p.pre_out + (size_t)m * K);
      float4 hv[kHeld], hg[kHeld], hb[kHeld];
      double ss = 0.0;
      auto sq = [](const float4& v) {
        return (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
      };
      if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
          const int i = tid + j * kKQThreads;
          const bool in = i < nvec;
          hv[j] = in ? __ldcg(xg + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          hg[j] = in ? __ldg(pg + i) : make_float4(0.f, 0.f, 0.f, 0.f);
          hb[j] = in ? __ldcg(bg + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < kHeld; ++j) ss += sq(hv[j]);
      } else {
        for (int i = tid; i < nvec; i += kKQThreads) ss += sq(__ldcg(xg + i));
      }
      ss = warp_sum(ss);
      if (lane == 0) red_f64[warp] = ss;
      __syncthreads();
      ss = 0.0;
#pragma unroll
      for (int i = 0; i < kKQWarps; ++i) ss += red_f64[i];
      const float r1 = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
      auto step = [&](int i, const float4& v, const float4& g, const float4& b) {
        float4 r;
        r.x = __fadd_rn(b.x, __fmul_rn(__fmul_rn(v.x, r1), g.x));
        r.y = __fadd_rn(b.y, __fmul_rn(__fmul_rn(v.y, r1), g.y));
        r.z = __fadd_rn(b.z, __fmul_rn(__fmul_rn(v.z, r1), g.z));
        r.w = __fadd_rn(b.w, __fmul_rn(__fmul_rn(v.w, r1), g.w));
        xs4[i] = r;
        if (blockIdx.x == 0) og[i] = r;
        ss2 += sq(r);
        return r;
      };
      if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
          const int i = tid + j * kKQThreads;
          if (i < nvec) hx[j] = step(i, hv[j], hg[j], hb[j]);
        }
      } else {
        for (int i = tid; i < nvec; i += kKQThreads) step(i, __ldcg(xg + i), __ldg(pg + i), __ldcg(bg + i));
      }
      if (gamma) {  // the second set of slots: the first may still be being read
        ss2 = warp_sum(ss2);
        if (lane == 0) red_f64[16 + warp] = ss2;
      }
      __syncthreads();
    }
    auto load_x = [&](int i) { return pre ? xs4[i] : __ldcg(xg + i); };
    if (gamma) {
      double ss = 0.0;
      if (pre) {
#pragma unroll
        for (int i = 0; i < kKQWarps; ++i) ss += red_f64[16 + i];
      } else {
        if (held) {
#pragma unroll
          for (int j = 0; j < kHeld; ++j)
            ss += (double)hx[j].x * hx[j].x + (double)hx[j].y * hx[j].y +
                  (double)hx[j].z * hx[j].z + (double)hx[j].w * hx[j].w;
        } else {
          for (int i = tid; i < nvec; i += kKQThreads) {
            const float4 v = load_x(i);
            ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
          }
        }
        ss = warp_sum(ss);
        if (lane == 0) red_f64[warp] = ss;
        __syncthreads();
        ss = 0.0;
#pragma unroll
        for (int i = 0; i < kKQWarps; ++i) ss += red_f64[i];
      }
      rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
    }
    // every group of 8 lanes owns one 32-element block; nvec is a multiple of 8.  v = the
    // normalised float4 number i of the row (zero beyond the row).
    auto quant4 = [&](int i, float4 v) {
      float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
      float sum = (v.x + v.y) + (v.z + v.w);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
      }
      const float inv = amax > 0.f ? 32512.0f / amax : 0.f;
      const float dx = amax / 32512.0f;
      const int q0 = __float2int_rn(v.x * inv), q1 = __float2int_rn(v.y * inv);
      const int q2 = __float2int_rn(v.z * inv), q3 = __float2int_rn(v.w * inv);
      if (i < nvec) {
        // 16-byte units of a chunk are XOR-swizzled by the chunk index so that
        // lanes reading the same unit of consecutive chunks hit distinct banks
        const int cb = i >> 4, wi = i & 15;
        const int si = (cb << 4) + ((((wi >> 2) ^ (cb >> 1)) & 3) << 2) + (wi & 3);
        xhi[si] = (uint32_t)((q0 >> 8) & 0xff) | ((uint32_t)((q1 >> 8) & 0xff) << 8) |
                 ((uint32_t)((q2 >> 8) & 0xff) << 16) | ((uint32_t)(q3 >> 8) << 24);
        xlo[si] = (uint32_t)(q0 & 0xff) | ((uint32_t)(q1 & 0xff) << 8) |
                 ((uint32_t)(q2 & 0xff) << 16) | ((uint32_t)q3 << 24);
        if ((lane & 7) == 0) {
          const int j = i >> 3;  // 32-element block index
          float* t = reinterpret_cast<float*>(xtab + (j >> 1));
          if (j & 1) {
            t[1] = FMT == 12 ? dx * 0.0625f : dx;
            t[3] = sum;
          } else {
            t[0] = dx;
            t[2] = sum;
          }
        }
      }
    };
    auto scaled = [&](float4 v, const float4& g) {
      if (gamma) {
        v.x = v.x * rinv * g.x;
        v.y = v.y * rinv * g.y;
        v.z = v.z * rinv * g.z;
        v.w = v.w * rinv * g.w;
      }
      return v;
    };
    if (held) {
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        const int i0 = warp * 32 + j * kKQThreads;  // warp-uniform: the shuffles stay whole
        if (i0 < nvec) quant4(i0 + lane, scaled(hx[j], hgm[j]));
      }
    } else {
      for (int i0 = warp * 32; i0 < nvec; i0 += kKQThreads) {
        const int i = i0 + lane;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nvec)
          v = scaled(load_x(i), gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + i) : v);
        quant4(i, v);
      }
    }
    __syncthreads();

    if (m > 0) {  // later tokens stream the weights again (from L2)
      tprod = t0 + warp;
      for (int n = 0; n < S && tprod < t1; ++n) produce();
    }

    // ---- streaming main loop (per warp) ---------------------------------------
    for (int t = t0 + warp; t < t1; t += kKQWarps) {
      const int sslot = slot_of(consumed);
      const uint32_t parity = (uint32_t)((consumed / S) & 1);
      int seg, row, nr;
      tile_at(t, seg, row, nr);
      mbar_wait(&bars[sslot], parity, p.status);
      const uint8_t* ws = wstage + (size_t)sslot * stage_bytes;

      float acc[kNS];
#pragma unroll
      for (int r = 0; r < kNS; ++r) acc[r] = 0.f;

      // whole passes: this lane's chunk is the same for every row of the tile
#pragma unroll 1
      for (int ps = 0; ps < npass; ++ps) {
        const int bc = ps * 32 + lane;
        uint32_t xh[16], xl[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ui = bc * 4 + (i ^ ((bc >> 1) & 3));
          const uint4 a = reinterpret_cast<const uint4*>(xhi)[ui];
          const uint4 b = reinterpret_cast<const uint4*>(xlo)[ui];
          xh[4 * i] = a.x; xh[4 * i + 1] = a.y; xh[4 * i + 2] = a.z; xh[4 * i + 3] = a.w;
          xl[4 * i] = b.x; xl[4 * i + 1] = b.y; xl[4 * i + 2] = b.z; xl[4 * i + 3] = b.w;
        }
        const float4 tab = xtab[bc];
        const int boff = FMT == 12 ? (bc >> 2) * 144 : bc * 68;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const uint8_t* base = ws + r * rowbytes + boff;
          acc[r] += FMT == 12 ? q4k_chunk(base, bc & 3, sel_main, xh, xl, tab) : q80_pair(base, xh, xl, tab);
        }
      }
      // leftover chunks: task index -> (row of the tile, chunk), no register reuse
#pragma unroll 1
      for (int u = 0; u < nrem_iter; ++u) {
        const int idx = u * 32 + lane;
        const bool ok = idx < rem * kRows;
        const int r = ok ? (int)__umulhi((uint32_t)idx, rem_magic) : 0;
        const int bc = npass * 32 + (ok ? idx - r * rem : 0);
        uint32_t xh[16], xl[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ui = bc * 4 + (i ^ ((bc >> 1) & 3));
          const uint4 a = reinterpret_cast<const uint4*>(xhi)[ui];
          const uint4 b = reinterpret_cast<const uint4*>(xlo)[ui];
          xh[4 * i] = a.x; xh[4 * i + 1] = a.y; xh[4 * i + 2] = a.z; xh[4 * i + 3] = a.w;
          xl[4 * i] = b.x; xl[4 * i + 1] = b.y; xl[4 * i + 2] = b.z; xl[4 * i + 3] = b.w;
        }
        const float4 tab = xtab[bc];
        const int boff = FMT == 12 ? (bc >> 2) * 144 : bc * 68;
        const uint8_t* base = ws + r * rowbytes + boff;
        float v = FMT == 12 ? q4k_chunk(base, bc & 3, q4k_sel(bc & 3), xh, xl, tab) : q80_pair(base, xh, xl, tab);
        v = ok ? v : 0.f;
#pragma unroll
        for (int rr = 0; rr < kRows; ++rr) acc[rr] += (r == rr) ? v : 0.f;
      }
      __syncwarp();
      if (tprod < t1) produce();

      // ---- reduce and store -----------------------------------------------------
      constexpr int kShift = kNS == 8 ? 2 : (kNS == 4 ? 3 : 4);
      const int slot = lane >> kShift;
      const bool writer = (lane & ((1 << kShift) - 1)) == 0;
      const float total = transpose_reduce_f<kNS>(acc, lane);
      if (!GU) {
        if (writer && slot < nr) {
          const KQSeg& sg = p.seg[seg];
          const size_t o = (size_t)m * sg.N + row + slot;
          float v = total;
          if (sg.residual) v += sg.residual[o];
          sg.y[o] = v;
        }
      } else {
        // gate row i is slot i, up row i is slot RT + i
        constexpr int kLanesPerSlot = 1 << kShift;
        const float up = __shfl_down_sync(0xffffffffu, total, RT * kLanesPerSlot);
        if (writer && slot < RT && slot < nr) {
          const size_t o = (size_t)m * p.seg[0].N + row + slot;
          p.seg[0].y[o] = gelu_tanh_f(total) * up;
        }
      }
      ++consumed;
    }
  }
}

// ---- batched path (16 tokens or more): a real contraction ------------------------------
//
// Both formats go through the kernel of kquant_mma.cu, which dequantises inside the tensor-core
// pipeline (weights and activations rounded to f16: ~4e-4 of max|y|, inside the 1e-3 bar).

// The optional pre-step (x' = base + rmsnorm(x) * pre_gamma, x' also written to pre_out) in
// front of a matvec call: inside the matvec kernel's prologue for a few tokens, inside the
// activation staging kernel of the batched path.
struct KQPre {
  const float* base;
  const float* gamma;
  float* out;
};

// One product of a batched call: y[M][N] = W x, plus a residual or, with glu set, times
// gelu_tanh of the gate values in `residual`.
struct KQBatchSeg {
  const uint8_t* blocks;
  long N;
  const float* residual;
  float* y;
  int glu;
};

// Q4_K or Q8_0 (K a multiple of 256), any M >= 1, several tensors against the same activations:
// the dequantiser is fused into the product kernel (kquant_mma.cu; split-K when there are few
// row tiles).  The activations of a pass are normalised, rounded and laid out once and shared
// by every tensor.
static int kq_batched_fused(hb200_ctx* ctx, int fmt, const KQBatchSeg* segs, int nseg, int K,
                            const float* d_x, int M, const KQPre& pre, const float* gamma,
                            float eps, cudaStream_t st) {
  ScratchUse use(ctx, st);  // staged activations, row scales, split-K partials, tickets
  // tokens per pass: the tensor time of a pass does not depend on it, the activation tile
  // and the accumulator do; K above 8192 keeps the 256-token tiles out of their scratch
  const int cap = K <= 8192 ? 256 : 128;
  for (int m0 = 0; m0 < M;) {
    const int left = M - m0;
    const int NT = left <= 64 ? 64 : (left <= 128 || cap == 128 ? 128 : 256);
    const int mc = left < NT ? left : NT;
    int rc = hb_gemm16_split_pre(ctx, 1, K, d_x + (size_t)m0 * K, mc,
                                 pre.gamma ? pre.base + (size_t)m0 * K : nullptr, pre.gamma,
                                 pre.gamma ? pre.out + (size_t)m0 * K : nullptr, gamma, eps, NT,
                                 st);
    if (rc != HB200_OK) return rc;
    // tensors without a GLU epilogue go into one launch, three at a time (their row tiles
    // add up, so small ones like k and v no longer leave most SMs idle); an up product
    // whose epilogue reads the gate product's output needs that launch finished first
    for (int s = 0; s < nseg;) {
      HbKqSeg run[3];
      int n = 0;
      do {
        const KQBatchSeg& g = segs[s];
        run[n++] = {g.blocks, g.N, g.y + (size_t)m0 * g.N,
                    g.residual ? g.residual + (size_t)m0 * g.N : nullptr, g.N, g.glu};
        ++s;
      } while (n < 3 && s < nseg && !segs[s].glu && !segs[s - 1].glu);
      rc = hb_kq_mma_run_multi(ctx, run, n, K, mc, NT, st, fmt);
      if (rc != HB200_OK) return rc;
    }
    m0 += mc;
  }
  return HB200_OK;
}

// ---- host side --------------------------------------------------------------------

static size_t kq_smem_bytes(int nslots, int rows, int K, int rowbytes, bool pre) {
  auto up128 = [](size_t v) { return (v + 127) & ~size_t(127); };
  size_t off = up128((size_t)nslots * 8);
  off += 32 * 8 + 2 * (size_t)K + (size_t)(K / 64) * 16 + (pre ? (size_t)K * 4 : 0);
  off = up128(off);
  return off + (size_t)nslots * rows * (size_t)rowbytes;
}

struct KQPlan {
  int rt, stages, nslots;
  size_t smem;
};

// Rows per tile and ring depth.  In order of preference:
//  (a) every tile of the CTA resident at once inside half of the SM's shared
//      memory, so that the next layer's kernel can sit beside this one and
//      prefetch (tallest tile wins);
//  (b) a ring of >= 2 stages inside half of the shared memory, most bytes in flight;
//  (c) the same inside the whole shared memory;  (d) whatever fits.
static bool kq_plan(const hb200_ctx* ctx, long rows, int K, int rowbytes, bool gu, bool pre,
                    KQPlan* out) {
  // One CTA per SM (the kernel wants ~166 registers per thread; capping it at the 80 that
  // would let two launches share an SM made it re-derive addresses and constants inside
  // the chunk loop for no net gain), so "half" below only keeps headroom for the L1.
  const size_t half = (size_t)ctx->smem_optin * 3 / 4, full = (size_t)ctx->smem_optin;
  KQPlan best = {0, 0, 0, 0};
  long best_bytes = -1;
  for (int pass = 0; pass < 4 && best.rt == 0; ++pass) {
    for (int rt = 4; rt >= 1; --rt) {
      const long tiles = (rows + rt - 1) / rt;
      const int grid = tiles < ctx->sm_count ? (int)tiles : ctx->sm_count;
      const int tpc = (int)((tiles + grid - 1) / grid);
      const int tpw = (tpc + kKQWarps - 1) / kKQWarps;
      const int srows = gu ? 2 * rt : rt;
      for (int st = (tpw < 4 ? tpw : 4); st >= 1; --st) {
        const int nslots = kKQWarps * st < tpc ? kKQWarps * st : tpc;
        const size_t sm = kq_smem_bytes(nslots, srows, K, rowbytes, pre);
        bool ok = false;
        if (pass == 0) ok = st == tpw && sm <= half;
        if (pass == 1) ok = st >= 2 && sm <= half;
        if (pass == 2) ok = (st >= 2 || st == tpw) && sm <= full;
        if (pass == 3) ok = sm <= full;
        const long inflight = (long)nslots * srows * rowbytes;
        if (ok && inflight > best_bytes) {
          best_bytes = inflight;
          best = {rt, st, nslots, sm};
        }
      }
      if (pass == 0 && best.rt) break;  // tallest fully resident tile
    }
  }
  if (!best.rt) return false;
  *out = best;
  return true;
}

template <int FMT, int RT, bool GU>
static int kq_launch(hb200_ctx* ctx, KQParams& p, size_t smem, cudaStream_t st) {
  auto kern = kquant_kernel<FMT, RT, GU>;
  {
    const int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(kern), smem);
    if (rc != HB200_OK) return rc;
  }
  const int grid = p.ntiles < ctx->sm_count ? p.ntiles : ctx->sm_count;
  HB_CUDA(launch_pdl(kern, dim3(grid), dim3(kKQThreads), smem, st, ctx->pdl, p));
  return HB200_OK;
}

template <int FMT, bool GU>
static int kq_dispatch(hb200_ctx* ctx, KQParams& p, const KQPlan& plan, cudaStream_t st) {
  switch (plan.rt) {
    case 1: return kq_launch<FMT, 1, GU>(ctx, p, plan.smem, st);
    case 2: return kq_launch<FMT, 2, GU>(ctx, p, plan.smem, st);
    case 3: return kq_launch<FMT, 3, GU>(ctx, p, plan.smem, st);
    default: return kq_launch<FMT, 4, GU>(ctx, p, plan.smem, st);
  }
}

static int kq_check(hb200_ctx* ctx, int fmt, int K, int M, const float* d_x) {
  HB_REQUIRE(ctx != nullptr, "kquant: null context");
  HB_REQUIRE(fmt == HB200_FMT_Q4_K || fmt == HB200_FMT_Q8_0,
             "kquant: format id %d is neither Q4_K (12) nor Q8_0 (8)", fmt);
  HB_REQUIRE(K > 0 && K % 256 == 0, "kquant: K=%d must be a positive multiple of 256", K);
  HB_REQUIRE(M >= 1 && M <= 4096, "kquant: M=%d outside 1..4096", M);
  HB_REQUIRE(d_x != nullptr && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0,
             "kquant: x must be non-null and 16-byte aligned");
  return HB200_OK;
}

static int kq_rowbytes(int fmt, int K) { return fmt == HB200_FMT_Q4_K ? K / 256 * 144 : K / 32 * 34; }

}  // namespace hb

using namespace hb;

static int kq_pre_check(const KQPre& pre, const float* d_x) {
  if (!pre.gamma) return HB200_OK;
  HB_REQUIRE(pre.base && pre.out, "kquant (pre-step): null pointer");
  HB_REQUIRE(((reinterpret_cast<uintptr_t>(pre.base) | reinterpret_cast<uintptr_t>(pre.gamma) |
               reinterpret_cast<uintptr_t>(pre.out)) & 15) == 0,
             "kquant (pre-step): arrays must be 16-byte aligned");
  HB_REQUIRE(pre.out != pre.base && pre.out != d_x,
             "kquant (pre-step): the output may not alias an input");
  return HB200_OK;
}

static int kq_forward_multi_impl(hb200_ctx* ctx, int fmt, const hb200_kquant_seg* segs, int nseg,
                                 int K, const float* d_x, int M, const KQPre& pre,
                                 const float* d_rms_gamma, float rms_eps, hb200_stream stream) {
  int rc = kq_check(ctx, fmt, K, M, d_x);
  if (rc) return rc;
  rc = kq_pre_check(pre, d_x);
  if (rc) return rc;
  HB_REQUIRE(segs && nseg >= 1 && nseg <= kKQMaxSeg, "kquant: nseg=%d outside 1..%d", nseg,
             kKQMaxSeg);
  long rows = 0;
  for (int s = 0; s < nseg; ++s) {
    HB_REQUIRE(segs[s].N >= 1 && segs[s].d_blocks && segs[s].d_y,
               "kquant: segment %d has N < 1 or a null pointer", s);
    HB_REQUIRE((reinterpret_cast<uintptr_t>(segs[s].d_blocks) & 15) == 0,
               "kquant: segment %d blocks must be 16-byte aligned", s);
    rows += segs[s].N;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M >= kKQBatchedFrom && !ctx->no_mma) {  // a real contraction: tensor-core path
    KQBatchSeg g[kKQMaxSeg];
    for (int s = 0; s < nseg; ++s)
      g[s] = {static_cast<const uint8_t*>(segs[s].d_blocks), segs[s].N, segs[s].d_residual,
              segs[s].d_y, 0};
    return kq_batched_fused(ctx, fmt, g, nseg, K, d_x, M, pre, d_rms_gamma, rms_eps, st);
  }
  HB_REQUIRE(M <= 64, "kquant: M=%d needs the batched path (HB200_NO_MMA is set)", M);
  if (M == 1) {  // one token: integer tensor-core matvec when the rows fit shared memory
    rc = hb_kq_mv_run(ctx, fmt, segs, nseg, K, 0, d_x, pre.base, pre.gamma, pre.out, d_rms_gamma,
                      rms_eps, st);
    if (rc <= 0) return rc;
  }
  const int rowbytes = kq_rowbytes(fmt, K);
  KQPlan plan;
  if (!kq_plan(ctx, rows, K, rowbytes, false, pre.gamma != nullptr, &plan)) {
    set_error("kquant: K=%d does not fit the shared-memory budget", K);
    return HB200_ERR_UNSUPPORTED;
  }
  KQParams p = {};
  int t = 0;
  for (int s = 0; s < nseg; ++s) {
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_blocks), segs[s].d_residual, segs[s].d_y,
                segs[s].N, t};
    t += (segs[s].N + plan.rt - 1) / plan.rt;
  }
  p.nseg = nseg;
  p.ntiles = t;
  p.K = K;
  p.M = M;
  p.stages = plan.stages;
  p.nslots = plan.nslots;
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.eps = rms_eps;
  p.status = ctx->d_status;
  p.pre_base = pre.base;
  p.pre_gamma = pre.gamma;
  p.pre_out = pre.out;
  return fmt == HB200_FMT_Q4_K ? kq_dispatch<12, false>(ctx, p, plan, st)
                               : kq_dispatch<8, false>(ctx, p, plan, st);
}

extern "C" int hb200_kquant_forward_multi(hb200_ctx* ctx, int fmt, const hb200_kquant_seg* segs,
                                          int nseg, int K, const float* d_x, int M,
                                          const float* d_rms_gamma, float rms_eps,
                                          hb200_stream stream) {
  return kq_forward_multi_impl(ctx, fmt, segs, nseg, K, d_x, M, KQPre{nullptr, nullptr, nullptr},
                               d_rms_gamma, rms_eps, stream);
}

extern "C" int hb200_kquant_forward_multi_pre(hb200_ctx* ctx, int fmt,
                                              const hb200_kquant_seg* segs, int nseg, int K,
                                              const float* d_o, int M, const float* d_pre_base,
                                              const float* d_pre_gamma, float* d_x_out,
                                              const float* d_rms_gamma, float rms_eps,
                                              hb200_stream stream) {
  HB_REQUIRE(d_pre_gamma != nullptr, "kquant (pre-step): null gamma");
  return kq_forward_multi_impl(ctx, fmt, segs, nseg, K, d_o, M,
                               KQPre{d_pre_base, d_pre_gamma, d_x_out}, d_rms_gamma, rms_eps,
                               stream);
}

extern "C" int hb200_kquant_forward(hb200_ctx* ctx, int fmt, const void* d_blocks, int K, int N,
                                    const float* d_x, int M, const float* d_rms_gamma,
                                    float rms_eps, const float* d_residual, float* d_y,
                                    hb200_stream stream) {
  hb200_kquant_seg s = {d_blocks, d_residual, d_y, N};
  return hb200_kquant_forward_multi(ctx, fmt, &s, 1, K, d_x, M, d_rms_gamma, rms_eps, stream);
}

static int kq_gateup_impl(hb200_ctx* ctx, int fmt, const void* d_blocks_gate,
                          const void* d_blocks_up, int K, int N, const float* d_x, int M,
                          const KQPre& pre, const float* d_rms_gamma, float rms_eps, float* d_y,
                          hb200_stream stream) {
  int rc = kq_check(ctx, fmt, K, M, d_x);
  if (rc) return rc;
  rc = kq_pre_check(pre, d_x);
  if (rc) return rc;
  HB_REQUIRE(N >= 1 && d_blocks_gate && d_blocks_up && d_y, "kquant gate/up: bad argument");
  HB_REQUIRE(((reinterpret_cast<uintptr_t>(d_blocks_gate) |
               reinterpret_cast<uintptr_t>(d_blocks_up)) & 15) == 0,
             "kquant gate/up: blocks must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M >= kKQBatchedFrom && !ctx->no_mma) {
    // both products on the tensor cores against one staging of the activations: the gate
    // product writes d_y, the up product's epilogue multiplies gelu_tanh(gate) in place
    const KQBatchSeg g[2] = {
        {static_cast<const uint8_t*>(d_blocks_gate), N, nullptr, d_y, 0},
        {static_cast<const uint8_t*>(d_blocks_up), N, d_y, d_y, 1}};
    return kq_batched_fused(ctx, fmt, g, 2, K, d_x, M, pre, d_rms_gamma, rms_eps, st);
  }
  HB_REQUIRE(M <= 64, "kquant gate/up: M=%d needs the batched path", M);
  if (M == 1) {
    const hb200_kquant_seg gs[2] = {{d_blocks_gate, nullptr, d_y, N}, {d_blocks_up, nullptr, d_y, N}};
    rc = hb_kq_mv_run(ctx, fmt, gs, 2, K, 1, d_x, pre.base, pre.gamma, pre.out, d_rms_gamma,
                      rms_eps, st);
    if (rc <= 0) return rc;
  }
  const int rowbytes = kq_rowbytes(fmt, K);
  KQPlan plan;
  if (!kq_plan(ctx, N, K, rowbytes, true, pre.gamma != nullptr, &plan)) {
    set_error("kquant gate/up: K=%d does not fit the shared-memory budget", K);
    return HB200_ERR_UNSUPPORTED;
  }
  KQParams p = {};
  p.seg[0] = {static_cast<const uint8_t*>(d_blocks_gate), nullptr, d_y, N, 0};
  p.seg[1] = {static_cast<const uint8_t*>(d_blocks_up), nullptr, d_y, N, 0};
  p.nseg = 2;
  p.ntiles = (N + plan.rt - 1) / plan.rt;
  p.K = K;
  p.M = M;
  p.stages = plan.stages;
  p.nslots = plan.nslots;
  p.x = d_x;
  p.gamma = d_rms_gamma;
  p.eps = rms_eps;
  p.status = ctx->d_status;
  p.pre_base = pre.base;
  p.pre_gamma = pre.gamma;
  p.pre_out = pre.out;
  return fmt == HB200_FMT_Q4_K ? kq_dispatch<12, true>(ctx, p, plan, st)
                               : kq_dispatch<8, true>(ctx, p, plan, st);
}

extern "C" int hb200_kquant_gateup_gelu(hb200_ctx* ctx, int fmt, const void* d_blocks_gate,
                                        const void* d_blocks_up, int K, int N, const float* d_x,
                                        int M, const float* d_rms_gamma, float rms_eps,
                                        float* d_y, hb200_stream stream) {
  return kq_gateup_impl(ctx, fmt, d_blocks_gate, d_blocks_up, K, N, d_x, M,
                        KQPre{nullptr, nullptr, nullptr}, d_rms_gamma, rms_eps, d_y, stream);
}

extern "C" int hb200_kquant_gateup_gelu_pre(hb200_ctx* ctx, int fmt, const void* d_blocks_gate,
                                            const void* d_blocks_up, int K, int N,
                                            const float* d_o, int M, const float* d_pre_base,
                                            const float* d_pre_gamma, float* d_x_out,
                                            const float* d_rms_gamma, float rms_eps, float* d_y,
                                            hb200_stream stream) {
  HB_REQUIRE(d_pre_gamma != nullptr, "kquant (pre-step): null gamma");
  return kq_gateup_impl(ctx, fmt, d_blocks_gate, d_blocks_up, K, N, d_o, M,
                        KQPre{d_pre_base, d_pre_gamma, d_x_out}, d_rms_gamma, rms_eps, d_y, stream);
}
