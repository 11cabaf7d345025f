// bitlinear_mv.cu -- one-token ternary (i2_s) x int8 matvec on the integer tensor-core
// instruction.
//
// Same contract as bitlinear.cu: acc[n] = sum_k t[n,k] * q[k] exactly in int32 (BitLinearSpec.forward,
// Hesper/Layers/BitLinearSpec.lean:65-91, on the int8 activations), y = ((float)acc * d) * s
// (+ residual); the reference's kernels for the layer are fusedBitLinearM1Kernel and its
// residual / RMSNorm / gate-up variants (Hesper/Layers/BitLinear.lean:297,361,447,553).
//
// The streaming kernel of bitlinear.cu spends ~3 thread instructions per weight (plane masks,
// dp4a, index arithmetic) and is bound by instruction issue, not by HBM.  Here:
//   * a CTA owns a contiguous range of rows that sits in shared memory at once, pulled in
//     16-row tiles by 1-D TMA bulk copies before griddepcontrol.wait; two launches fit on an
//     SM, so the next layer's weights load while this layer computes;
//   * a 32-byte i2_s group holds 128 weights as four 2-bit planes (Hesper/Layers/
//     BitLinearSpec.lean:43-60): plane s of a packed word is w & (0xC0 >> 2s) per byte, the
//     code scaled by 4^(3-s), which is a valid u8 operand of mma.sync.m16n8k32 (u8 x s8 ->
//     s32).  One AND per 16 weights and row, one MMA per plane, group and 16 rows;
//   * the eight B columns carry the int8 activations of the eight (group, plane) pairs of 256
//     consecutive weights, each MMA seeing zeros in the other columns, so all eight MMAs of a
//     256-weight column block add into ONE accumulator fragment that lives across the whole
//     K range of the warp; the plane factors are shifted out once per tile (exact: every
//     column sum is a multiple of its factor), value = code - 1 is restored by subtracting
//     sum(q) once per row;
//   * a lane's 8 bytes of a row are one LDS.64 (the k order inside a plane is permuted
//     identically on both operands), and with that permutation the B fragments of a column
//     block are simply its 256 int8 activations in natural order;
//   * warps own column blocks; their int32 row partials meet in shared memory by atomicAdd
//     (integer: any order gives the same bits);
//   * ROPE variant (fused q/k/v of one token): the rows of every q and k head are dealt out in
//     the order d, d + D/2, d + 1, d + 1 + D/2, ... so that a CTA holds both elements of every
//     rotation pair, and the epilogue applies the NeoX rotation (the arithmetic of rope.cuh, in
//     double) and writes q as f32 and k / v as f16 straight into the KV cache: the separate
//     RoPE + KV-write launch of a decode step disappears.
#include "common.cuh"

namespace hb {

constexpr int kBmWarps = 10;
constexpr int kBmThreads = kBmWarps * 32;
constexpr int kBmMaxTiles = 16;
constexpr int kBmMaxSeg = 4;
constexpr int kBmHeld = 3;  // groups of 8 activations a thread keeps in registers

struct BmSeg {
  const uint8_t* w;
  const float* scale;
  const float* residual;
  float* y;
  int32_t* acc;
  int N;
  int row0;  // first virtual row of the segment
};

struct BmParams {
  BmSeg seg[kBmMaxSeg];
  int nseg;
  int rows;      // virtual rows: all segments, or 2N for gate/up (tiles of 8 gate + 8 up rows)
  int K;
  int rows_cap;  // most rows any CTA owns, rounded up to 16
  int rows_max;  // most rows any CTA owns
  int per, rem;  // units per CTA and how many CTAs own one more (unit: row, or gate/up tile)
  const float* x;
  const float* gamma;
  float eps;
  float* act_scale;
  uint32_t* status;
  // ROPE variant: segments are q, k, v of ONE token of one sequence
  const double2* rope_table;  // [D/2] (cos, sin) of the token's angles
  const int32_t* pos;         // [1] the token's position
  __half* k_cache;            // [Hkv][slots][D]
  __half* v_cache;
  int D, slots, ring;
};

// Rows are K/4 bytes, a multiple of 64: laid end to end, the same byte of every row would fall
// into the same shared-memory bank and the eight rows a warp reads at once would queue up.
// 32 bytes of padding per row put consecutive rows 8 banks apart (two wavefronts per LDS.64 of
// a warp, the minimum for 256 bytes).
__host__ __device__ inline int bm_row_stride(int K) { return (K >> 2) + 32; }

struct BmSmem {
  size_t part, xq, w, total;
};
__host__ __device__ inline BmSmem bm_smem(int rows_cap, int rows_max, int K) {
  BmSmem s;
  size_t off = 128 + 256 + 128;  // tile barriers | f64 reduction scratch | amax / sum(q) scratch
  s.part = off;
  off += (size_t)rows_cap * sizeof(int32_t);
  off = (off + 15) & ~size_t(15);
  s.xq = off;
  off += (size_t)K;
  off = (off + 127) & ~size_t(127);
  s.w = off;
  s.total = off + (size_t)rows_max * (size_t)bm_row_stride(K);
  return s;
}

__device__ __forceinline__ void bm_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Row `o` of a q / k segment in the ROPE row order -> the tensor's own row: inside a head the
// virtual rows 2j, 2j + 1 are the rotation pair (j, j + D/2).
__device__ __forceinline__ int bm_rope_row(int o, int D) {
  const int h = o / D, j = o - h * D;
  return h * D + (j >> 1) + (j & 1) * (D >> 1);
}

// GU: fused ReLU^2 GLU of a gate and an up tensor (tiles of 8 gate rows + 8 up rows).
// ROPE: q / k / v of one token with the rotation and the KV-cache write in the epilogue.
template <bool GU, bool ROPE>
__global__ void __launch_bounds__(kBmThreads, 2) bl_mv_kernel(const __grid_constant__ BmParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K;
  const int rowbytes = K >> 2;
  const int nblk = K >> 8;  // column blocks of 256 weights (two i2_s groups)

  pdl_trigger();

  // rows of this CTA: the first `rem` CTAs own one unit more
  const int b = blockIdx.x;
  const int u0 = b * p.per + min(b, p.rem);
  const int u1 = u0 + p.per + (b < p.rem ? 1 : 0);
  const int v0 = GU ? u0 << 4 : (ROPE ? u0 << 1 : u0), v1 = GU ? u1 << 4 : (ROPE ? u1 << 1 : u1);
  const int nrows = v1 - v0;
  const int ntiles = (nrows + 15) >> 4;

  const BmSmem L = bm_smem(p.rows_cap, p.rows_max, K);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);             // [kBmMaxTiles]
  double* red = reinterpret_cast<double*>(smem + 128);            // [16]
  uint32_t* red_u = reinterpret_cast<uint32_t*>(smem + 384);      // [16] warp maxima
  int32_t* red_i = reinterpret_cast<int32_t*>(smem + 384 + 64);   // [16] warp sums of q
  int32_t* part = reinterpret_cast<int32_t*>(smem + L.part);      // [rows_cap]
  uint8_t* xq = smem + L.xq;                                      // [K] int8 activations
  uint8_t* wbase = smem + L.w;

  // warp w starts the copies of tiles w, w + 10, ...: one bulk copy per row (rows are padded in
  // shared memory), the 16 rows of a tile issued by 16 lanes
  const int stride = bm_row_stride(K);
  {
    const uint64_t pol = policy_evict_first();
    for (int j = warp; j < ntiles; j += kBmWarps) {
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
          const int i = lane & 7;  // rows 0..7 of the tile are gate rows, 8..15 up rows
          src = p.seg[lane >> 3].w + ((size_t)(a >> 1) + i) * rowbytes;
        } else {
          int sg = 0;
#pragma unroll
          for (int s = 1; s < kBmMaxSeg; ++s)
            if (s < p.nseg && vr >= p.seg[s].row0) sg = s;
          int o = vr - p.seg[sg].row0;
          if (ROPE && sg < 2) o = bm_rope_row(o, p.D);
          src = p.seg[sg].w + (size_t)o * rowbytes;
        }
        bulk_g2s_stream(wbase + (size_t)(16 * j + lane) * stride, src, (uint32_t)rowbytes,
                        &bars[j], pol);
      }
    }
  }
  if (tid < 16) {
    red[tid] = 0.0;
    red_u[tid] = 0u;
    red_i[tid] = 0;
  }
  for (int i = tid; i < p.rows_cap; i += kBmThreads) part[i] = 0;

  // everything else that does not depend on the previous kernel: the tensors' scales, the norm
  // weights of the activations this thread will hold
  float wscale[GU ? 2 : kBmMaxSeg];
#pragma unroll
  for (int s = 0; s < (GU ? 2 : kBmMaxSeg); ++s) wscale[s] = s < p.nseg ? __ldg(p.seg[s].scale) : 0.f;
  const int n8 = K >> 3;  // groups of 8 consecutive activations
  const bool held = n8 <= kBmHeld * kBmThreads;
  const float* const gamma = p.gamma;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 hg[kBmHeld][2];
#pragma unroll
  for (int j = 0; j < kBmHeld; ++j) {
    const int i = tid + j * kBmThreads;
    const bool in = held && gamma && i < n8;
    hg[j][0] = in ? __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i) : zero4;
    hg[j][1] = in ? __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i + 1) : zero4;
  }
  __syncthreads();  // barriers initialised, scratch cleared

  // column blocks and tiles of this warp
  const int nslot = nblk < kBmWarps ? nblk : kBmWarps;
  const int slot = warp % nslot;
  const int tgroups = kBmWarps / nslot;
  const int tg = warp / nslot;
  const bool active = tg < tgroups;

  pdl_wait();

  // ---- activation prologue: (RMSNorm), per-token absmax, int8 -- bit for bit the arithmetic
  //      of the streaming kernel: d = amax / 127, inv = 127 / amax (IEEE divisions),
  //      q = rint(x * inv) ------------------------------------------------------------------
  float dtok;
  int sumq_total;
  {
    // x and the residual were written by the kernel this one depends on, while this kernel was
    // already resident: they are read past L1 (ld.global.cg), never through the read-only path,
    // whose lines an earlier kernel on this SM may have filled before the writes.
    const float4* xg = reinterpret_cast<const float4*>(p.x);
    float4 hx[kBmHeld][2];
#pragma unroll
    for (int j = 0; j < kBmHeld; ++j) {
      const int i = tid + j * kBmThreads;
      const bool in = held && i < n8;
      hx[j][0] = in ? __ldcg(xg + 2 * i) : zero4;
      hx[j][1] = in ? __ldcg(xg + 2 * i + 1) : zero4;
    }
    float rinv = 1.f;
    if (gamma) {
      auto sq = [](const float4& v) {
        return (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
      };
      double ss = 0.0;
      if (held) {
#pragma unroll
        for (int j = 0; j < kBmHeld; ++j) ss += sq(hx[j][0]) + sq(hx[j][1]);
      } else {
        for (int i = tid; i < 2 * n8; i += kBmThreads) ss += sq(__ldcg(xg + i));
      }
      ss = warp_sum(ss);
      if (lane == 0) red[warp] = ss;
      __syncthreads();
      ss = 0.0;
#pragma unroll
      for (int i = 0; i < kBmWarps; ++i) ss += red[i];
      rinv = (float)(1.0 / sqrt(ss / (double)K + (double)p.eps));
    }
    auto normed = [&](float4 v, const float4& gq) {
      if (gamma) {
        v.x = __fmul_rn(__fmul_rn(v.x, rinv), gq.x);
        v.y = __fmul_rn(__fmul_rn(v.y, rinv), gq.y);
        v.z = __fmul_rn(__fmul_rn(v.z, rinv), gq.z);
        v.w = __fmul_rn(__fmul_rn(v.w, rinv), gq.w);
      }
      return v;
    };
    auto amax4 = [](const float4& v) {
      return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    };
    auto load_normed = [&](int i4) {  // float4 number i4 of the normalised row (not held)
      return normed(__ldcg(xg + i4),
                    gamma ? __ldg(reinterpret_cast<const float4*>(gamma) + i4) : zero4);
    };
    float amax = 0.f;
    if (held) {
#pragma unroll
      for (int j = 0; j < kBmHeld; ++j) {
        hx[j][0] = normed(hx[j][0], hg[j][0]);
        hx[j][1] = normed(hx[j][1], hg[j][1]);
        amax = fmaxf(amax, fmaxf(amax4(hx[j][0]), amax4(hx[j][1])));
      }
    } else {
      for (int i = tid; i < 2 * n8; i += kBmThreads) amax = fmaxf(amax, amax4(load_normed(i)));
    }
    // non-negative floats order like their bit patterns: one redux per warp
    const uint32_t wmax = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
    if (lane == 0) red_u[warp] = wmax;
    __syncthreads();
    {
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < kBmWarps; ++i) mx = max(mx, red_u[i]);
      amax = __uint_as_float(mx);
    }
    dtok = __fdiv_rn(amax, 127.0f);
    const float inv = amax == 0.f ? 0.f : __fdiv_rn(127.0f, amax);
    int sumq = 0;
    auto quant8 = [&](int i, const float4& a, const float4& c) {
      const int q0 = __float2int_rn(__fmul_rn(a.x, inv)), q1 = __float2int_rn(__fmul_rn(a.y, inv));
      const int q2 = __float2int_rn(__fmul_rn(a.z, inv)), q3 = __float2int_rn(__fmul_rn(a.w, inv));
      const int q4 = __float2int_rn(__fmul_rn(c.x, inv)), q5 = __float2int_rn(__fmul_rn(c.y, inv));
      const int q6 = __float2int_rn(__fmul_rn(c.z, inv)), q7 = __float2int_rn(__fmul_rn(c.w, inv));
      sumq += ((q0 + q1) + (q2 + q3)) + ((q4 + q5) + (q6 + q7));
      uint2 w;
      w.x = __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
      w.y = __byte_perm(__byte_perm(q4, q5, 0x0040), __byte_perm(q6, q7, 0x0040), 0x5410);
      *reinterpret_cast<uint2*>(xq + 8 * (size_t)i) = w;  // natural order = B fragment order
    };
    if (held) {
#pragma unroll
      for (int j = 0; j < kBmHeld; ++j) {
        const int i = tid + j * kBmThreads;
        if (i < n8) quant8(i, hx[j][0], hx[j][1]);
      }
    } else {
      for (int i = tid; i < n8; i += kBmThreads) quant8(i, load_normed(2 * i), load_normed(2 * i + 1));
    }
    sumq = __reduce_add_sync(0xffffffffu, sumq);
    if (lane == 0) red_i[warp] = sumq;
    if (tid == 0 && blockIdx.x == 0 && p.act_scale) p.act_scale[0] = dtok;
    // the warp that started a tile's copies sees them land; after the barrier everybody knows
    for (int j = warp; j < ntiles; j += kBmWarps) mbar_wait(&bars[j], 0, p.status);
    __syncthreads();
    sumq_total = 0;
#pragma unroll
    for (int i = 0; i < kBmWarps; ++i) sumq_total += red_i[i];
  }

  // ---- the products ---------------------------------------------------------------------------
  if (active) {
    // plane factors of the two columns whose accumulators this lane owns (columns 2t, 2t+1:
    // planes 0,1 for even t, planes 2,3 for odd t)
    const int sh0 = (t & 1) ? 2 : 6, sh1 = (t & 1) ? 0 : 4;
    for (int blk = slot; blk < nblk; blk += nslot) {
      // B operand: column g = (group g >> 2 of the block, plane g & 3); this lane's 8 bytes of it
      const uint2 bx = *reinterpret_cast<const uint2*>(xq + (size_t)blk * 256 + 8 * lane);
      uint32_t bq[8][2];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        bq[q][0] = q == g ? bx.x : 0u;
        bq[q][1] = q == g ? bx.y : 0u;
      }
      for (int j = tg; j < ntiles; j += tgroups) {
        const int lrA = min(16 * j + g, nrows - 1), lrB = min(16 * j + g + 8, nrows - 1);
        const uint8_t* rA = wbase + (size_t)lrA * stride + (size_t)blk * 64 + 8 * t;
        const uint8_t* rB = wbase + (size_t)lrB * stride + (size_t)blk * 64 + 8 * t;
        // the two groups of the block own disjoint columns: separate fragments halve the
        // dependency chain of the eight MMAs, their sum is the block's fragment
        int c[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0};
        {
          const uint2 wa = *reinterpret_cast<const uint2*>(rA), wb = *reinterpret_cast<const uint2*>(rB);
          const uint2 xa = *reinterpret_cast<const uint2*>(rA + 32), xb = *reinterpret_cast<const uint2*>(rB + 32);
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const uint32_t mk = 0xC0C0C0C0u >> (2 * s);
            bm_mma(c, wa.x & mk, wb.x & mk, wa.y & mk, wb.y & mk, bq[s][0], bq[s][1]);
            bm_mma(c2, xa.x & mk, xb.x & mk, xa.y & mk, xb.y & mk, bq[4 + s][0], bq[4 + s][1]);
          }
        }
        int vA = ((c[0] + c2[0]) >> sh0) + ((c[1] + c2[1]) >> sh1);
        int vB = ((c[2] + c2[2]) >> sh0) + ((c[3] + c2[3]) >> sh1);
        vA += __shfl_xor_sync(0xffffffffu, vA, 1);
        vB += __shfl_xor_sync(0xffffffffu, vB, 1);
        vA += __shfl_xor_sync(0xffffffffu, vA, 2);
        vB += __shfl_xor_sync(0xffffffffu, vB, 2);
        if (t < 2) atomicAdd(&part[16 * j + g + 8 * t], t ? vB : vA);
      }
    }
  }
  __syncthreads();

  // ---- value = code - 1: subtract sum(q); scale, epilogue, store ----------------------------
  if (ROPE) {
    int pos = __ldcg(p.pos);
    int slot = p.ring ? pos % p.slots : pos;
    slot = slot < 0 ? 0 : (slot >= p.slots ? p.slots - 1 : slot);
    const int D = p.D, half = D >> 1;
    for (int lr = 2 * tid; lr < nrows; lr += 2 * kBmThreads) {  // a pair of virtual rows
      const int vr = v0 + lr;
      int sg = 0;
#pragma unroll
      for (int s = 1; s < kBmMaxSeg; ++s)
        if (s < p.nseg && vr >= p.seg[s].row0) sg = s;
      const BmSeg& S = p.seg[sg];
      const int o = vr - S.row0;  // even
      float ws = wscale[0];
#pragma unroll
      for (int s = 1; s < kBmMaxSeg; ++s) ws = sg == s ? wscale[s] : ws;
      const float y0 = __fmul_rn(__fmul_rn((float)(part[lr] - sumq_total), dtok), ws);
      const float y1 = __fmul_rn(__fmul_rn((float)(part[lr + 1] - sumq_total), dtok), ws);
      const int h = o / D, j = o - h * D;
      if (sg < 2) {
        // rotation pair (d, d + D/2) of head h: the arithmetic of rope_kv_element
        const int d = j >> 1;
        const double2 a = p.rope_table[d];
        const double x0 = y0, x1 = y1;
        const float r0 = (float)(x0 * a.x - x1 * a.y), r1 = (float)(x0 * a.y + x1 * a.x);
        if (sg == 0) {
          S.y[h * D + d] = r0;
          S.y[h * D + d + half] = r1;
        } else {
          __half* dst = p.k_cache + ((size_t)h * p.slots + slot) * D;
          dst[d] = __float2half_rn(r0);
          dst[d + half] = __float2half_rn(r1);
        }
      } else {
        __half* dst = p.v_cache + ((size_t)h * p.slots + slot) * D;
        *reinterpret_cast<__half2*>(dst + j) = __floats2half2_rn(y0, y1);
      }
    }
  } else if (!GU) {
    for (int lr = tid; lr < nrows; lr += kBmThreads) {
      const int total = part[lr] - sumq_total;
      const int vr = v0 + lr;
      int sg = 0;
#pragma unroll
      for (int s = 1; s < kBmMaxSeg; ++s)
        if (s < p.nseg && vr >= p.seg[s].row0) sg = s;
      const BmSeg& S = p.seg[sg];
      const int o = vr - S.row0;
      if (S.acc) S.acc[o] = total;
      float ws = wscale[0];
#pragma unroll
      for (int s = 1; s < kBmMaxSeg; ++s) ws = sg == s ? wscale[s] : ws;
      float v = __fmul_rn(__fmul_rn((float)total, dtok), ws);
      if (S.residual) v = __fadd_rn(v, __ldcg(S.residual + o));
      S.y[o] = v;
    }
  } else {
    for (int i = tid; i < (nrows >> 1); i += kBmThreads) {
      const int lr = ((i >> 3) << 4) + (i & 7);  // gate row; its up row is 8 further
      const float gt = __fmul_rn(__fmul_rn((float)(part[lr] - sumq_total), dtok), wscale[0]);
      const float up = __fmul_rn(__fmul_rn((float)(part[lr + 8] - sumq_total), dtok), wscale[1]);
      const float r = gt > 0.f ? gt : 0.f;
      p.seg[0].y[(v0 >> 1) + i] = __fmul_rn(__fmul_rn(r, r), up);
    }
  }
}

}  // namespace hb

using namespace hb;

// One token through the tensor-core ternary matvec.  HB200_OK when the launch was made, 1 when
// the shape is outside what this kernel covers (the caller takes the streaming kernel), < 0 on
// error.
int hb_bl_mv_run(hb200_ctx* ctx, const hb200_bitlinear_seg* segs, int nseg, int K, int gu,
                 const float* d_x, const float* gamma, float eps, float* d_act_scale,
                 cudaStream_t st, const HbRope* rope) {
  if (ctx->mv_mode == 0 || (K & 255)) return 1;
  long rows = 0;
  if (gu) {
    if (nseg != 2 || segs[0].N != segs[1].N || (segs[0].N & 7)) return 1;
    rows = 2L * segs[0].N;
  } else {
    for (int s = 0; s < nseg; ++s) rows += segs[s].N;
  }
  if (rope) {  // q, k, v of one token: whole heads, pairs of rows are the unit of the split
    if (gu || nseg != 3 || rope->D < 2 || (rope->D & 1) || segs[0].N % rope->D ||
        segs[1].N % rope->D || segs[2].N != segs[1].N)
      return 1;
  }
  if (rows > (1L << 30)) return 1;
  const int ushift = gu ? 4 : (rope ? 1 : 0);  // rows per unit of the split: 16, 2 or 1
  const long units = rows >> ushift;
  const int grid = (int)(units < ctx->sm_count ? units : ctx->sm_count);
  const int per = (int)(units / grid), rem = (int)(units % grid);
  const int rows_max = (per + (rem ? 1 : 0)) << ushift;
  const int rows_cap = (rows_max + 15) & ~15;
  if (rows_cap > 16 * kBmMaxTiles) return 1;
  const size_t smem = bm_smem(rows_cap, rows_max, K).total;
  if (smem > (size_t)ctx->smem_optin) return 1;
  if (ctx->mv_mode == 1 && 2 * (smem + 1024) > ctx->smem_per_sm) return 1;

  BmParams p = {};
  int r0 = 0;
  for (int s = 0; s < nseg; ++s) {
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_packed), segs[s].d_scale,
                segs[s].d_residual, segs[s].d_y, segs[s].d_acc, segs[s].N, gu ? 0 : r0};
    r0 += segs[s].N;
  }
  p.nseg = nseg;
  p.rows = (int)rows;
  p.K = K;
  p.rows_cap = rows_cap;
  p.rows_max = rows_max;
  p.per = per;
  p.rem = rem;
  p.x = d_x;
  p.gamma = gamma;
  p.eps = eps;
  p.act_scale = d_act_scale;
  p.status = ctx->d_status;
  if (rope) {
    p.rope_table = reinterpret_cast<const double2*>(rope->table);
    p.pos = rope->pos;
    p.k_cache = static_cast<__half*>(rope->k_cache);
    p.v_cache = static_cast<__half*>(rope->v_cache);
    p.D = rope->D;
    p.slots = rope->slots;
    p.ring = rope->ring;
  }
  void (*kern)(BmParams) = gu ? bl_mv_kernel<true, false>
                              : (rope ? bl_mv_kernel<false, true> : bl_mv_kernel<false, false>);
  int rc = hb_func_smem(ctx, reinterpret_cast<const void*>(kern), smem);
  if (rc != HB200_OK) return rc;
  HB_CUDA(launch_pdl(kern, dim3(grid), dim3(kBmThreads), smem, st, ctx->pdl, p));
  return HB200_OK;
}
