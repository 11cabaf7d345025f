// kquant_mv.cu -- one-token GGUF Q4_K / Q8_0 matvec on the integer tensor-core instruction.
//
// Same contract as kquant.cu (y[n] = sum_k dequant(W)[n,k] * x[k], block formats of
// Hesper/Quantization/Q4_K_M.lean:13-52,120-144 and Hesper/Layers/Linear.lean:6187-6223; the
// reference's kernels for these layers are mulMvQ4KF32Kernel, Hesper/WGSL/MulMvQ4K.lean:46,
// and fusedQ8_0LinearKernel, Hesper/Layers/Linear.lean:6192), one token per call.
//
// A launch on the dependent chain of a decode step costs what follows griddepcontrol.wait:
// everything that does not need the activations is done before it.
//   * a CTA owns a contiguous range of rows, small enough to sit in shared memory at once;
//     the warps pull 16-row tiles with 1-D TMA bulk copies, one mbarrier per tile (one copy per
//     tile, or one per row where the rows are padded against bank conflicts).
//     With 320 threads, <= 96 registers and <= ~113 KB of shared memory two launches fit on an
//     SM, so the next layer's kernel loads (and prepares) its weights while this one computes.
//     The kernel has no pipeline of its own -- all rows land before the products start -- so
//     next to a kernel that fills its SM's shared memory the load is not hidden; the host
//     routes shapes here only where sharing an SM is possible and measured faster;
//   * still before the wait, the 6-bit scales and mins of every Q4_K super-block are decoded
//     and written back over the 12 packed bytes as one word per 64-weight chunk
//     {scale_even, scale_odd, min_even, min_odd}; d and dmin move to a side array;
//   * after the wait the CTA quantises the activations once, per 32 elements to 16 bits,
//     x ~ dx * (256*hi + lo) with hi and lo signed bytes, and lays the two byte planes out as
//     the B fragments of mma.sync.m16n8k32 (u8/s8 x s8 -> s32);
//   * A = 16 rows x one 32-weight sub-block, nibbles separated by one AND per four weights
//     (the high nibble is used in place, its factor 16 folded into the activation scale; Q8_0
//     quants are fed as they are).  A lane's 8 bytes of a row are one LDS.64: the k order
//     inside a sub-block is permuted identically on both operands;
//   * the eight B columns carry {hi, lo} of the four 64-weight chunks of a 256-weight
//     super-block, each chunk's MMA seeing zeros in the other chunks' columns.  The eight MMAs
//     of a super-block so accumulate into two fragments in which lane t of a quad holds chunk
//     t: every lane post-processes one sub-block pair of two rows;
//   * a warp owns super-block columns (warp w: super-blocks w, w+10, ...); per-row partials
//     of the warps meet in shared memory; one barrier, fixed summation order.
#include "common.cuh"

namespace hb {

constexpr int kMvWarps = 10;
constexpr int kMvThreads = kMvWarps * 32;
constexpr int kMvMaxTiles = 16;  // 16-row tiles a CTA may hold
constexpr int kMvMaxSeg = 4;

struct MvSeg {
  const uint8_t* w;
  const float* residual;
  float* y;
  int N;
  int row0;  // first virtual row of the segment
};

struct MvParams {
  MvSeg seg[kMvMaxSeg];
  int nseg;
  int rows;      // virtual rows: all segments, or 2N for gate/up (tiles of 8 gate + 8 up rows)
  int K;
  int rows_cap;  // most rows any CTA owns, rounded up to 16
  int rows_max;  // most rows any CTA owns
  int per, rem;  // units per CTA and how many CTAs own one more (unit: row, or gate/up tile)
  int nslot;     // partial-sum slots: min(super-blocks, warps)
  const float* x;
  const float* gamma;
  float eps;
  uint32_t* status;
  const float* pre_base;
  const float* pre_gamma;
  float* pre_out;
};

// Shared-memory carve-up, the same arithmetic on host and device.
struct MvSmem {
  size_t part, side, xfrag, xtab, xs, w, total;
};
// Bytes between two rows in shared memory.  A warp's fragment load touches eight rows at the same
// column (eight words per row for Q4_K): with a stride of 8 words (mod 32) the rows spread over
// all banks, with 0 (K = 2048, 10240, ...) they would all start on the same bank.  The padding
// is a multiple of 16 bytes, so a row still is a legal bulk-copy destination.
__host__ __device__ inline int mv_row_stride(int rowbytes) {
  const int w = rowbytes >> 2;
  return rowbytes + 4 * ((((8 - w) % 32) + 32) % 32);
}
// Words between two rows of the {d, dmin} side array: eight rows at one column collide only when
// the stride is a multiple of 8 words.
__host__ __device__ inline int mv_side_stride(int nsb) { return (nsb & 7) ? nsb : nsb + 1; }

__host__ __device__ inline MvSmem mv_smem(int fmt, int nslot, int rows_cap, int rows_max, int K,
                                          int rowbytes, bool pre) {
  const int nsb = K >> 8;
  MvSmem s;
  size_t off = 128 + 256;  // tile barriers, reduction scratch
  s.part = off;
  off += (size_t)nslot * rows_cap * sizeof(float);
  s.side = off;
  if (fmt == 12) off += (size_t)rows_max * mv_side_stride(nsb) * sizeof(uint32_t);
  off = (off + 15) & ~size_t(15);
  s.xfrag = off;
  off += (size_t)nsb * 512;
  s.xtab = off;
  off += (size_t)nsb * 64;
  s.xs = off;
  if (pre) off += (size_t)K * sizeof(float);
  off = (off + 127) & ~size_t(127);
  s.w = off;
  s.total = off + (size_t)rows_max * mv_row_stride(rowbytes);
  return s;
}

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The four bytes of v as floats (I2F with a byte selector, no masking).
__device__ __forceinline__ void mv_u8x4_to_f(uint32_t v, float& a, float& b, float& c, float& d) {
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
      "mov.b32 {t0, t1, t2, t3}, %4;\n\t"
      "cvt.rn.f32.u8 %0, t0;\n\t"
      "cvt.rn.f32.u8 %1, t1;\n\t"
      "cvt.rn.f32.u8 %2, t2;\n\t"
      "cvt.rn.f32.u8 %3, t3;\n\t}"
      : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
      : "r"(v));
}

__device__ __forceinline__ float mv_gelu_tanh(float x) {
  // Hesper/Layers/FusedFFNSpec.lean:42-45
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(u));
}

// Per-lane constants of a super-block column: B fragments of the four chunks (zero where the
// lane's column belongs to another chunk) and the activation scales / sums of the chunk whose
// accumulators the lane owns.
struct MvCol {
  uint32_t b[4][4];  // [chunk][even k0..3, even k4..7, odd k0..3, odd k4..7]
  float dxe, dxo, Se, So;
};

// One Q4_K unit: rows (g, g+8) of a tile x one super-block.  The lane's header word is the
// pre-decoded {scale_even, scale_odd, min_even, min_odd} of chunk t, dd = half2 {d, dmin}.
__device__ __forceinline__ void mv_unit_q4k(const uint8_t* rA, const uint8_t* rB, uint32_t ddA,
                                            uint32_t ddB, int t, const MvCol& col, float& vA,
                                            float& vB) {
  int ce[4] = {0, 0, 0, 0}, co[4] = {0, 0, 0, 0};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint2 wa = *reinterpret_cast<const uint2*>(rA + 16 + 32 * c + 8 * t);
    const uint2 wb = *reinterpret_cast<const uint2*>(rB + 16 + 32 * c + 8 * t);
    mma_u8s8(ce, wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu,
             col.b[c][0], col.b[c][1]);
    mma_u8s8(co, wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u,
             col.b[c][2], col.b[c][3]);
  }
  const uint32_t hA = *reinterpret_cast<const uint32_t*>(rA + 4 * t);
  const uint32_t hB = *reinterpret_cast<const uint32_t*>(rB + 4 * t);
  auto row_value = [&](uint32_t h, uint32_t dd, int hi_e, int lo_e, int hi_o, int lo_o) {
    float scl, sch, ml, mh;
    mv_u8x4_to_f(h, scl, sch, ml, mh);
    const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&dd));
    const float fe = (float)(hi_e * 256 + lo_e);
    const float fo = (float)(hi_o * 256 + lo_o);
    const float main = fmaf(sch * col.dxo, fo, (scl * col.dxe) * fe);
    const float mins = fmaf(mh, col.So, ml * col.Se);
    return fmaf(d.x, main, -(d.y * mins));
  };
  vA = row_value(hA, ddA, ce[0], ce[1], co[0], co[1]);
  vB = row_value(hB, ddB, ce[2], ce[3], co[2], co[3]);
}

// One Q8_0 unit: block b of the 272-byte unit sits at byte 34 b; its 32 quants start 2 bytes
// in, so even blocks are read as three words and realigned, odd blocks are word aligned.
__device__ __forceinline__ void mv_unit_q80(const uint8_t* rA, const uint8_t* rB, int t,
                                            const MvCol& col, float& vA, float& vB) {
  int ce[4] = {0, 0, 0, 0}, co[4] = {0, 0, 0, 0};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t* ea = reinterpret_cast<const uint32_t*>(rA + 68 * c + 8 * t);
    const uint32_t* eb = reinterpret_cast<const uint32_t*>(rB + 68 * c + 8 * t);
    const uint32_t a0 = ea[0], a1 = ea[1], a2 = ea[2];
    const uint32_t b0 = eb[0], b1 = eb[1], b2 = eb[2];
    const uint32_t* oa = reinterpret_cast<const uint32_t*>(rA + 68 * c + 36 + 8 * t);
    const uint32_t* ob = reinterpret_cast<const uint32_t*>(rB + 68 * c + 36 + 8 * t);
    mma_s8s8(ce, __funnelshift_r(a0, a1, 16), __funnelshift_r(b0, b1, 16),
             __funnelshift_r(a1, a2, 16), __funnelshift_r(b1, b2, 16), col.b[c][0], col.b[c][1]);
    mma_s8s8(co, oa[0], ob[0], oa[1], ob[1], col.b[c][2], col.b[c][3]);
  }
  auto row_value = [&](const uint8_t* r, int hi_e, int lo_e, int hi_o, int lo_o) {
    const float de = __half2float(*reinterpret_cast<const __half*>(r + 68 * t));
    const float dq = __half2float(*reinterpret_cast<const __half*>(r + 68 * t + 34));
    const float fe = (float)(hi_e * 256 + lo_e);
    const float fo = (float)(hi_o * 256 + lo_o);
    return fmaf(dq * col.dxo, fo, (de * col.dxe) * fe);
  };
  vA = row_value(rA, ce[0], ce[1], co[0], co[1]);
  vB = row_value(rB, ce[2], ce[3], co[2], co[3]);
}

// FMT: 12 = Q4_K (144-byte super-blocks), 8 = Q8_0 (eight 34-byte blocks per 256 weights).
template <int FMT, bool GU>
__global__ void __launch_bounds__(kMvThreads, 2) kq_mv_kernel(const __grid_constant__ MvParams p) {
  constexpr int kUnit = FMT == 12 ? 144 : 272;  // bytes of 256 weights
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K;
  const int nsb = K >> 8;
  const int rowbytes = nsb * kUnit;
  const int stride = mv_row_stride(rowbytes);
  const int sstride = mv_side_stride(nsb);

  pdl_trigger();

  // rows of this CTA: the first `rem` CTAs own one unit more (a unit is a row, or a 16-row
  // gate/up tile)
  const int b = blockIdx.x;
  const int u0 = b * p.per + min(b, p.rem);
  const int u1 = u0 + p.per + (b < p.rem ? 1 : 0);
  const int v0 = GU ? u0 << 4 : u0, v1 = GU ? u1 << 4 : u1;
  const int nrows = v1 - v0;
  const int ntiles = (nrows + 15) >> 4;

  const bool pre = p.pre_gamma != nullptr;
  const MvSmem L = mv_smem(FMT, p.nslot, p.rows_cap, p.rows_max, K, rowbytes, pre);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);            // [kMvMaxTiles]
  double* red = reinterpret_cast<double*>(smem + 128);           // [2][16]
  float* part = reinterpret_cast<float*>(smem + L.part);         // [nslot][rows_cap]
  uint32_t* side = reinterpret_cast<uint32_t*>(smem + L.side);   // [rows][nsb] half2 {d, dmin}
  uint8_t* xfrag = smem + L.xfrag;                               // [nsb][32 lanes][16]
  float* xtab = reinterpret_cast<float*>(smem + L.xtab);         // [nsb][dx[8], sum[8]]
  float* xs = reinterpret_cast<float*>(smem + L.xs);             // [K] with the pre-step
  uint8_t* wbase = smem + L.w;

  // Warp w starts the copies of tiles w, w + 10, ...: one copy per tile (or per segment piece)
  // from lane 0 where rows sit back to back, else one copy per row from lanes 0..15.
  if (stride != rowbytes) {
    const uint64_t pol = policy_evict_first();
    for (int j = warp; j < ntiles; j += kMvWarps) {
      const int a = v0 + 16 * j;
      const int e = min(a + 16, v1);
      if (lane == 0) {
        mbar_init(&bars[j], 1);
        fence_mbar_init();
        mbar_arrive_expect_tx(&bars[j], (uint32_t)(e - a) * rowbytes);
      }
      __syncwarp();
      if (lane < e - a) {
        const int vr = a + lane;  // virtual row
        const uint8_t* src;
        if (GU) {
          // rows 0..7 of the tile are gate rows, 8..15 the up rows of the same outputs
          src = p.seg[lane >> 3].w + ((size_t)(a >> 1) + (lane & 7)) * rowbytes;
        } else {
          int sg = 0;
#pragma unroll
          for (int s = 1; s < kMvMaxSeg; ++s)
            if (s < p.nseg && vr >= p.seg[s].row0) sg = s;
          src = p.seg[sg].w + (size_t)(vr - p.seg[sg].row0) * rowbytes;
        }
        bulk_g2s_stream(wbase + (size_t)(16 * j + lane) * stride, src, (uint32_t)rowbytes,
                        &bars[j], pol);
      }
    }
  } else if (lane == 0) {
    const uint64_t pol = policy_evict_first();
    for (int j = warp; j < ntiles; j += kMvWarps) {
      mbar_init(&bars[j], 1);
      fence_mbar_init();
      const int a = v0 + 16 * j;
      const int e = min(a + 16, v1);
      mbar_arrive_expect_tx(&bars[j], (uint32_t)(e - a) * rowbytes);
      uint8_t* dst = wbase + (size_t)(16 * j) * rowbytes;
      if (GU) {
        const size_t r = (size_t)(a >> 1);  // first gate/up row of the tile
        bulk_g2s_stream(dst, p.seg[0].w + r * rowbytes, 8u * rowbytes, &bars[j], pol);
        bulk_g2s_stream(dst + 8 * (size_t)rowbytes, p.seg[1].w + r * rowbytes, 8u * rowbytes,
                        &bars[j], pol);
      } else if (p.nseg == 1) {
        bulk_g2s_stream(dst, p.seg[0].w + (size_t)a * rowbytes, (uint32_t)(e - a) * rowbytes,
                        &bars[j], pol);
      } else {
#pragma unroll
        for (int s = 0; s < kMvMaxSeg; ++s) {
          if (s < p.nseg) {
            const int lo = max(a, p.seg[s].row0), hi = min(e, p.seg[s].row0 + p.seg[s].N);
            if (lo < hi)
              bulk_g2s_stream(dst + (size_t)(lo - a) * rowbytes,
                              p.seg[s].w + (size_t)(lo - p.seg[s].row0) * rowbytes,
                              (uint32_t)(hi - lo) * rowbytes, &bars[j], pol);
          }
        }
      }
    }
  }
  if (tid < 32) red[tid] = 0.0;
  __syncthreads();  // barriers initialised before anyone polls them

  // which super-block columns and which tiles this warp works on
  const int nslot = p.nslot;      // min(nsb, warps)
  const int slot = warp % nslot;  // super-blocks slot, slot + nslot, ...
  const int tgroups = kMvWarps / nslot;
  const int tg = warp / nslot;    // tiles tg, tg + tgroups, ...
  const bool active = tg < tgroups;

  // ---- before the dependency: the tiles land, Q4_K headers are decoded in place ----------
  if (active) {
    for (int j = tg; j < ntiles; j += tgroups) {
      mbar_wait(&bars[j], 0, p.status);
      if (FMT == 12) {
        const int lrA = min(16 * j + g, nrows - 1), lrB = min(16 * j + g + 8, nrows - 1);
        // scale / min selectors of chunk t (Hesper/Quantization/Q4_K_M.lean:120-144)
        const bool upper = t >= 2;
        const uint32_t sh = (uint32_t)(t & 1) * 16u;
        const uint32_t mask_lo = upper ? 0x0F0Fu : 0x3F3Fu;
        const uint32_t mask_hi = upper ? 0x3030u : 0u;
        const uint32_t m_extra = upper ? 4u : 0u;
        for (int sb = slot; sb < nsb; sb += nslot) {
          uint8_t* rA = wbase + (size_t)lrA * stride + (size_t)sb * kUnit;
          uint8_t* rB = wbase + (size_t)lrB * stride + (size_t)sb * kUnit;
          const uint4 hA = *reinterpret_cast<const uint4*>(rA);
          const uint4 hB = *reinterpret_cast<const uint4*>(rB);
          auto chunk_word = [&](const uint4& h) {
            const uint32_t wa = upper ? h.w : h.y;
            const uint32_t wm = upper ? h.w : h.z;
            const uint32_t sc2 = ((wa >> sh) & mask_lo) | ((h.y >> (sh + 2)) & mask_hi);
            const uint32_t m2 = ((wm >> (sh + m_extra)) & mask_lo) | ((h.z >> (sh + 2)) & mask_hi);
            return sc2 | (m2 << 16);
          };
          const uint32_t wA = chunk_word(hA), wB = chunk_word(hB);
          __syncwarp();  // every lane of the quad has read the packed header
          *reinterpret_cast<uint32_t*>(rA + 4 * t) = wA;
          *reinterpret_cast<uint32_t*>(rB + 4 * t) = wB;
          if (t == 0) {
            side[lrA * sstride + sb] = hA.x;
            side[lrB * sstride + sb] = hB.x;
          }
          __syncwarp();
        }
      }
    }
  }

  // A thread owns groups of 8 consecutive activations (two float4); four lanes share a
  // 32-element block.  One group per thread (K <= 2560) stays in registers from their first read
  // to the quantisation.  Norm weights are constants of the model: fetch them ahead of the
  // dependency.
  constexpr int kHeld = 1;
  const int n8 = K >> 3;
  const bool held = n8 <= kHeld * kMvThreads;
  const float* const gamma = p.gamma;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 hgm[kHeld][2];
#pragma unroll
  for (int j = 0; j < kHeld; ++j) {
    const int i = tid + j * kMvThreads;
    const bool in = held && gamma && i < n8;
    hgm[j][0] = in ? __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i) : zero4;
    hgm[j][1] = in ? __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i + 1) : zero4;
  }

  pdl_wait();

  // ---- activation prologue: (pre-step), (RMSNorm), per-32 block 16-bit quantisation --------
  {
    // x, the pre-step's base and the residual were written by the kernel this one depends on,
    // while this kernel was already resident: they are read past L1 (ld.global.cg), never through
    // the read-only path, whose lines an earlier kernel on this SM may have filled before.
    const float4* xg = reinterpret_cast<const float4*>(p.x);
    float rinv = 1.f;
    double ss2 = 0.0;
    float4 hx[kHeld][2];
#pragma unroll
    for (int j = 0; j < kHeld; ++j) {
      const int i = tid + j * kMvThreads;
      const bool in = held && !pre && i < n8;
      hx[j][0] = in ? __ldcg(xg + 2 * i) : zero4;
      hx[j][1] = in ? __ldcg(xg + 2 * i + 1) : zero4;
    }
    auto sq = [](const float4& v) {
      return (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    };
    if (pre) {
      // x' = base + rmsnorm(x) * pre_gamma, operation order of the stand-alone kernel
      const float4* pg = reinterpret_cast<const float4*>(p.pre_gamma);
      const float4* bg = reinterpret_cast<const float4*>(p.pre_base);
      float4* og = reinterpret_cast<float4*>(p.pre_out);
      float4 hv[kHeld][2], hg[kHeld][2], hb[kHeld][2];
      double ss = 0.0;
      if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
          const int i = tid + j * kMvThreads;
          const bool in = i < n8;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            hv[j][h] = in ? __ldcg(xg + 2 * i + h) : zero4;
            hg[j][h] = in ? __ldg(pg + 2 * i + h) : zero4;
            hb[j][h] = in ? __ldcg(bg + 2 * i + h) : zero4;
          }
        }
#pragma unroll
        for (int j = 0; j < kHeld; ++j) ss += sq(hv[j][0]) + sq(hv[j][1]);
      } else {
        for (int i = tid; i < 2 * n8; i += kMvThreads) ss += sq(__ldcg(xg + i));
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = 0.0;
#pragma unroll
      for (int i = 0; i < kMvWarps; ++i) ss += red[i];
      const float r1 = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
      auto step = [&](int i, const float4& v, const float4& gq, const float4& bq) {
        float4 r;
        r.x = __fadd_rn(bq.x, __fmul_rn(__fmul_rn(v.x, r1), gq.x));
        r.y = __fadd_rn(bq.y, __fmul_rn(__fmul_rn(v.y, r1), gq.y));
        r.z = __fadd_rn(bq.z, __fmul_rn(__fmul_rn(v.z, r1), gq.z));
        r.w = __fadd_rn(bq.w, __fmul_rn(__fmul_rn(v.w, r1), gq.w));
        reinterpret_cast<float4*>(xs)[i] = r;
        if (blockIdx.x == 0) og[i] = r;
        ss2 += sq(r);
        return r;
      };
      if (held) {
#pragma unroll
        for (int j = 0; j < kHeld; ++j) {
          const int i = tid + j * kMvThreads;
          if (i < n8) {
            hx[j][0] = step(2 * i, hv[j][0], hg[j][0], hb[j][0]);
            hx[j][1] = step(2 * i + 1, hv[j][1], hg[j][1], hb[j][1]);
          }
        }
      } else {
        for (int i = tid; i < 2 * n8; i += kMvThreads)
          step(i, __ldcg(xg + i), __ldg(pg + i), __ldcg(bg + i));
      }
      if (gamma) {
        ss2 = warp_sum(ss2);
        if (lane == 0) red[16 + warp] = ss2;
      }
      __syncthreads();
    }
    auto load_x = [&](int i) {
      return pre ? reinterpret_cast<const float4*>(xs)[i] : __ldcg(xg + i);
    };
    if (gamma) {
      double ss = 0.0;
      if (pre) {
#pragma unroll
        for (int i = 0; i < kMvWarps; ++i) ss += red[16 + i];
      } else {
        if (held) {
#pragma unroll
          for (int j = 0; j < kHeld; ++j) ss += sq(hx[j][0]) + sq(hx[j][1]);
        } else {
          for (int i = tid; i < 2 * n8; i += kMvThreads) ss += sq(load_x(i));
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        ss = 0.0;
#pragma unroll
        for (int i = 0; i < kMvWarps; ++i) ss += red[i];
      }
      rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
    }
    // Group i of the normalised row (elements 8i..8i+7; zero beyond the row) -> bytes where
    // the MMA's B operand wants them: column 2c + plane of chunk c is lane group g = 2c +
    // plane, a lane's 16 bytes are {even sub-block elements 8t..8t+3, 8t+4..8t+7, odd
    // sub-block likewise}.  q + 128 = 256*hi + (lo + 128): hi is byte 1 of the biased value,
    // lo its byte 0 with the top bit flipped.
    auto quant8 = [&](int i, const float4& a, const float4& b) {
      float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                         fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
      float sum = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
#pragma unroll
      for (int o = 1; o < 4; o <<= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
      }
      const float inv = amax > 0.f ? __fdividef(32512.0f, amax) : 0.f;
      const float dx = amax * (1.0f / 32512.0f);
      const uint32_t q0 = (uint32_t)__float2int_rn(fmaf(a.x, inv, 128.f));
      const uint32_t q1 = (uint32_t)__float2int_rn(fmaf(a.y, inv, 128.f));
      const uint32_t q2 = (uint32_t)__float2int_rn(fmaf(a.z, inv, 128.f));
      const uint32_t q3 = (uint32_t)__float2int_rn(fmaf(a.w, inv, 128.f));
      const uint32_t q4 = (uint32_t)__float2int_rn(fmaf(b.x, inv, 128.f));
      const uint32_t q5 = (uint32_t)__float2int_rn(fmaf(b.y, inv, 128.f));
      const uint32_t q6 = (uint32_t)__float2int_rn(fmaf(b.z, inv, 128.f));
      const uint32_t q7 = (uint32_t)__float2int_rn(fmaf(b.w, inv, 128.f));
      uint2 lo, hi;
      lo.x = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410) ^
             0x80808080u;
      lo.y = __byte_perm(__byte_perm(q4, q5, 0x0040), __byte_perm(q6, q7, 0x0040), 0x5410) ^
             0x80808080u;
      hi.x = __byte_perm(__byte_perm(q0, q1, 0x0051), __byte_perm(q2, q3, 0x0051), 0x5410);
      hi.y = __byte_perm(__byte_perm(q4, q5, 0x0051), __byte_perm(q6, q7, 0x0051), 0x5410);
      if (i < n8) {
        const int e = i << 3;  // first element
        const int sbi = e >> 8, c = (e >> 6) & 3, odd = (e >> 5) & 1, tq = (e >> 3) & 3;
        uint8_t* dst = xfrag + (size_t)sbi * 512 + ((8 * c + tq) << 4) + (odd << 3);
        *reinterpret_cast<uint2*>(dst) = hi;       // lane group 2c
        *reinterpret_cast<uint2*>(dst + 64) = lo;  // lane group 2c + 1
        if (tq == 0) {
          const int j = (e >> 5) & 7;
          xtab[sbi * 16 + j] = (FMT == 12 && odd) ? dx * 0.0625f : dx;
          xtab[sbi * 16 + 8 + j] = sum;
        }
      }
    };
    auto scaled = [&](float4 v, const float4& gq) {
      if (gamma) {
        v.x = v.x * rinv * gq.x;
        v.y = v.y * rinv * gq.y;
        v.z = v.z * rinv * gq.z;
        v.w = v.w * rinv * gq.w;
      }
      return v;
    };
    if (held) {
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        const int i0 = warp * 32 + j * kMvThreads;  // warp-uniform: the shuffles stay whole
        if (i0 < n8) quant8(i0 + lane, scaled(hx[j][0], hgm[j][0]), scaled(hx[j][1], hgm[j][1]));
      }
    } else {
      for (int i0 = warp * 32; i0 < n8; i0 += kMvThreads) {
        const int i = i0 + lane;
        float4 va = zero4, vb = zero4;
        if (i < n8) {
          const float4* g4 = reinterpret_cast<const float4*>(gamma);
          va = scaled(load_x(2 * i), gamma ? __ldg(g4 + 2 * i) : zero4);
          vb = scaled(load_x(2 * i + 1), gamma ? __ldg(g4 + 2 * i + 1) : zero4);
        }
        quant8(i, va, vb);
      }
    }
  }
  __syncthreads();

  // ---- the products ---------------------------------------------------------------------------
  if (active) {
    const int cB = g >> 1;  // the chunk whose activations this lane's B column carries
    for (int sb = slot; sb < nsb; sb += nslot) {
      MvCol col;
      {
        const uint4 bf = *reinterpret_cast<const uint4*>(xfrag + (size_t)sb * 512 + lane * 16);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const bool mine = c == cB;
          col.b[c][0] = mine ? bf.x : 0u;
          col.b[c][1] = mine ? bf.y : 0u;
          col.b[c][2] = mine ? bf.z : 0u;
          col.b[c][3] = mine ? bf.w : 0u;
        }
        const float2 dx = *reinterpret_cast<const float2*>(xtab + sb * 16 + 2 * t);
        const float2 sm = *reinterpret_cast<const float2*>(xtab + sb * 16 + 8 + 2 * t);
        col.dxe = dx.x;
        col.dxo = dx.y;
        col.Se = sm.x;
        col.So = sm.y;
      }
      // two tiles per iteration: their dependency chains are independent and interleave
      auto unit = [&](int j, float& vA, float& vB) {
        const int lrA = min(16 * j + g, nrows - 1), lrB = min(16 * j + g + 8, nrows - 1);
        const uint8_t* rA = wbase + (size_t)lrA * stride + (size_t)sb * kUnit;
        const uint8_t* rB = wbase + (size_t)lrB * stride + (size_t)sb * kUnit;
        if (FMT == 12)
          mv_unit_q4k(rA, rB, side[lrA * sstride + sb], side[lrB * sstride + sb], t, col, vA, vB);
        else
          mv_unit_q80(rA, rB, t, col, vA, vB);
      };
      auto finish = [&](int j, float vA, float vB) {
        // the four chunks of the super-block sit on the four lanes of the quad
        vA += __shfl_xor_sync(0xffffffffu, vA, 1);
        vB += __shfl_xor_sync(0xffffffffu, vB, 1);
        vA += __shfl_xor_sync(0xffffffffu, vA, 2);
        vB += __shfl_xor_sync(0xffffffffu, vB, 2);
        if (t < 2) {
          float* dst = part + (size_t)slot * p.rows_cap + 16 * j + g + 8 * t;
          const float v = t ? vB : vA;
          *dst = sb == slot ? v : *dst + v;
        }
      };
      int j = tg;
      for (; j + tgroups < ntiles; j += 2 * tgroups) {
        float vA0, vB0, vA1, vB1;
        unit(j, vA0, vB0);
        unit(j + tgroups, vA1, vB1);
        finish(j, vA0, vB0);
        finish(j + tgroups, vA1, vB1);
      }
      for (; j < ntiles; j += tgroups) {
        float vA, vB;
        unit(j, vA, vB);
        finish(j, vA, vB);
      }
    }
  }
  __syncthreads();

  // ---- sum the slots in fixed order, epilogue, store ---------------------------------------
  if (!GU) {
    for (int lr = tid; lr < nrows; lr += kMvThreads) {
      float v = 0.f;
      for (int s = 0; s < nslot; ++s) v += part[(size_t)s * p.rows_cap + lr];
      const int vr = v0 + lr;
      int sg = 0;
#pragma unroll
      for (int s = 1; s < kMvMaxSeg; ++s)
        if (s < p.nseg && vr >= p.seg[s].row0) sg = s;
      const MvSeg& S = p.seg[sg];
      const int o = vr - S.row0;
      if (S.residual) v += __ldcg(S.residual + o);
      S.y[o] = v;
    }
  } else {
    for (int i = tid; i < (nrows >> 1); i += kMvThreads) {
      const int lr = ((i >> 3) << 4) + (i & 7);  // gate row; its up row is 8 further
      float gt = 0.f, up = 0.f;
      for (int s = 0; s < nslot; ++s) {
        gt += part[(size_t)s * p.rows_cap + lr];
        up += part[(size_t)s * p.rows_cap + lr + 8];
      }
      p.seg[0].y[(v0 >> 1) + i] = mv_gelu_tanh(gt) * up;
    }
  }
}

}  // namespace hb

using namespace hb;

// One token through the tensor-core matvec.  Returns HB200_OK when the launch was made, 1 when
// the shape is outside what this kernel covers (the caller then takes the streaming kernel),
// < 0 on error.
int hb_kq_mv_run(hb200_ctx* ctx, int fmt, const hb200_kquant_seg* segs, int nseg, int K, int gu,
                 const float* d_x, const float* pre_base, const float* pre_gamma, float* pre_out,
                 const float* gamma, float eps, cudaStream_t st) {
  if (ctx->mv_mode == 0) return 1;
  const int nsb = K >> 8;
  const int rowbytes = fmt == HB200_FMT_Q4_K ? nsb * 144 : nsb * 272;
  long rows = 0;
  if (gu) {
    if (nseg != 2 || segs[0].N != segs[1].N || (segs[0].N & 7)) return 1;
    rows = 2L * segs[0].N;
  } else {
    for (int s = 0; s < nseg; ++s) rows += segs[s].N;
  }
  if (rows > (1L << 30)) return 1;
  const long units = gu ? rows >> 4 : rows;  // what is dealt to the CTAs
  const int grid = (int)(units < ctx->sm_count ? units : ctx->sm_count);
  const int per = (int)(units / grid), rem = (int)(units % grid);
  const int rows_max = (per + (rem ? 1 : 0)) << (gu ? 4 : 0);
  const int rows_cap = (rows_max + 15) & ~15;
  if (rows_cap > 16 * kMvMaxTiles) return 1;
  const int nslot = nsb < kMvWarps ? nsb : kMvWarps;
  const size_t smem =
      mv_smem(fmt, nslot, rows_cap, rows_max, K, rowbytes, pre_gamma != nullptr).total;
  // Measured on B200: where two launches fit on an SM and a CTA has at least three tiles, this
  // kernel beats the streaming kernel (K=2560 N=10240: 5.0 vs 6.0 us in a ring of distinct
  // matrices); inside a decode step, between kernels of other kinds, the streaming kernel
  // was the faster one for the small projections, so those stay with it.
  if (smem > (size_t)ctx->smem_optin) return 1;
  if (ctx->mv_mode == 1 && (2 * (smem + 1024) > ctx->smem_per_sm || rows_max < 48)) return 1;

  MvParams p = {};
  int r0 = 0;
  for (int s = 0; s < nseg; ++s) {
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_blocks), segs[s].d_residual, segs[s].d_y,
                segs[s].N, gu ? 0 : r0};
    r0 += segs[s].N;
  }
  p.nseg = nseg;
  p.rows = (int)rows;
  p.K = K;
  p.rows_cap = rows_cap;
  p.rows_max = rows_max;
  p.per = per;
  p.rem = rem;
  p.nslot = nslot;
  p.x = d_x;
  p.gamma = gamma;
  p.eps = eps;
  p.status = ctx->d_status;
  p.pre_base = pre_base;
  p.pre_gamma = pre_gamma;
  p.pre_out = pre_out;

  void (*kern)(MvParams) = nullptr;
  if (fmt == HB200_FMT_Q4_K) kern = gu ? kq_mv_kernel<12, true> : kq_mv_kernel<12, false>;
  else kern = gu ? kq_mv_kernel<8, true> : kq_mv_kernel<8, false>;
  int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(kern), smem);
  if (rc != HB200_OK) return rc;
  HB_CUDA(launch_pdl(kern, dim3(grid), dim3(kMvThreads), smem, st, ctx->pdl, p));
  return HB200_OK;
}
