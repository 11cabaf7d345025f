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
//   bitlinear_mma_kernel  one CTA per 128 weight rows:
//     * packed rows arrive by per-row TMA bulk copies in chunks of 8 groups (1024 weights)
//       on a 3-deep ring;
//     * warps 0-7 expand one 128-wide group per step from 2-bit codes to unsigned bytes
//       (0,1,2) directly into the A-operand layout (16 ALU pairs and 4 x 16-byte stores per
//       thread and step) -- the expansion is the only per-weight work left on the SM; they
//       hand stages over through mbarriers only, there is no CTA-wide barrier in the loop;
//     * warp 8 drives the copies and issues 4 tcgen05.mma (M=128, N=64 tokens, K=32 each) per
//       step from one thread, operands described by shared-memory matrix descriptors (no
//       swizzle), D[128x64] int32 in 64 TMEM columns; tcgen05.commit releases the stage;
//     * epilogue: 4 warps read their 32 TMEM lanes (tcgen05.ld 32x32b), subtract sum(q) per
//       token (value = code - 1), scale and store.
// Every mbarrier wait is bounded; on expiry the kernel still releases its tensor memory.
#include "common.cuh"

namespace hb {

constexpr int kMmaThreads = 256;
constexpr int kMmaRows = 128;    // weight rows per CTA = MMA M
constexpr int kMmaTokens = 64;   // MMA N
constexpr int kChunkGroups = 8;  // 128-weight groups per packed chunk
constexpr int kPkStages = 3, kExStages = 4;
constexpr int kPkRowBytes = kChunkGroups * 32;          // 256 packed bytes per row and chunk
constexpr int kPkBytes = kMmaRows * kPkRowBytes;        // 32 KB
constexpr int kABytes = kMmaRows * 128;                 // 16 KB expanded A stage
constexpr int kBBytes = kMmaTokens * 128;               // 8 KB B stage
constexpr int kMmaSmem = 1024 + kPkStages * kPkBytes + kExStages * (kABytes + kBBytes);

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
  MmaSeg seg[4];
  int nseg, K, M;
  const uint8_t* xq;   // [K/128][64 tokens x 128 bytes, core-matrix layout]
  const float* d;      // [64] activation scales
  const int32_t* sumq; // [64]
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
};

__global__ void __launch_bounds__(256) quant_act_kernel(const __grid_constant__ QuantParams p) {
  __shared__ double red_d[8];
  __shared__ uint32_t red_u[8];
  __shared__ int red_i[8];
  extern __shared__ __align__(16) float xs[];  // [K]
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, nvec = K >> 2;
  auto dst_of = [&](int i) {  // float4 index -> byte offset of its 4 int8 in the operand layout
    const int k = i << 2;
    return (size_t)(k >> 7) * kBBytes + (size_t)(m >> 3) * 1024 + (size_t)((k & 127) >> 4) * 128 +
           (size_t)(m & 7) * 16 + (k & 15);
  };
  if (m >= p.M) {  // padding token of the 64-wide tile
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
      const float4 v = __ldg(xg + i);
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
      const float4 v = __ldg(xg + i);
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

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes,
// LBO = byte distance between core matrices adjacent in K, SBO = between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  return d;                // base offset 0, layout type 0 (no swizzle)
}

// Instruction descriptor for kind::i8: D = s32, A = u8, B = s8, both K-major, N = 64, M = 128.
constexpr uint32_t kIdescI8 = (2u << 4) | (0u << 7) | (1u << 10) | ((kMmaTokens >> 3) << 17) |
                              ((kMmaRows >> 4) << 24);

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(kIdescI8), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

// Bounded wait with a tighter cap than the streaming kernels use: a tile's whole life is a
// few microseconds, so ~1e5 polls already means something is broken.  Once a wait has
// failed the later ones are skipped, so a broken launch ends quickly.
__device__ __forceinline__ bool mma_wait(bool ok, uint64_t* bar, uint32_t parity, uint32_t* status) {
  if (!ok) return false;
#pragma unroll 1
  for (uint32_t it = 0; it < (1u << 17); ++it)
    if (mbar_try_wait(bar, parity)) return true;
  atomicOr(status, kStatusMbarTimeout);
  return false;
}

__global__ void __launch_bounds__(kMmaThreads + 32, 1)
    bitlinear_mma_kernel(const __grid_constant__ MmaParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, rowbytes = K >> 2, ngroups = K >> 7;
  const int nchunks = (ngroups + kChunkGroups - 1) / kChunkGroups;
  constexpr int kExpWarps = kMmaThreads / 32;  // warps 0..7 expand, warp 8 drives TMA and MMA

  // control block, then packed ring, then expanded stages (1 KB aligned for the descriptors)
  uint64_t* pk_full = reinterpret_cast<uint64_t*>(smem);  // [3] packed chunk landed (tx bytes)
  uint64_t* pk_free = pk_full + kPkStages;                 // [3] all expander warps done with it
  uint64_t* a_full = pk_free + kPkStages;                  // [4] A stage written by all expanders
  uint64_t* b_full = a_full + kExStages;                   // [4] B stage landed (tx bytes)
  uint64_t* st_free = b_full + kExStages;                  // [4] MMAs that read the stage finished
  uint64_t* done = st_free + kExStages;                    // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  float* sd = reinterpret_cast<float*>(smem + 256);        // [64]
  int* ssum = reinterpret_cast<int*>(smem + 512);          // [64]
  uint8_t* pk = smem + 1024;
  uint8_t* ex = pk + kPkStages * kPkBytes;

  // tile -> (segment, first row)
  int seg = 0;
#pragma unroll
  for (int s = 1; s < 4; ++s)
    if (s < p.nseg && (int)blockIdx.x >= p.seg[s].tile0) seg = s;
  const MmaSeg& sg = p.seg[seg];
  const int row0 = ((int)blockIdx.x - sg.tile0) * kMmaRows;
  const int nrows = min(kMmaRows, sg.N - row0);

  if (tid == 0) {
    for (int i = 0; i < kPkStages; ++i) {
      mbar_init(&pk_full[i], 1);
      mbar_init(&pk_free[i], kExpWarps);
    }
    for (int i = 0; i < kExStages; ++i) {
      mbar_init(&a_full[i], kExpWarps);
      mbar_init(&b_full[i], 1);
      mbar_init(&st_free[i], 1);
    }
    mbar_init(done, 1);
    fence_mbar_init();
  }
  if (warp == kExpWarps) {  // 64 TMEM columns: the 128 x 64 int32 accumulator
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 64;" ::"r"(
        smem_u32(tmem_slot)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bool ok = true;

  if (warp == kExpWarps) {
    // ================= control warp: TMA producer and MMA issuer =========================
    const uint64_t pol = policy_evict_first();
    // packed chunk c: one bulk copy per row (rows past the tensor's end repeat its last row)
    auto issue_chunk = [&](int c) {
      const int st = c % kPkStages;
      const int g0 = c * kChunkGroups;
      const uint32_t bytes = (uint32_t)min(kChunkGroups, ngroups - g0) * 32u;
      if (lane == 0) mbar_arrive_expect_tx(&pk_full[st], bytes * kMmaRows);
      __syncwarp();
#pragma unroll
      for (int i = 0; i < kMmaRows / 32; ++i) {
        const int r = lane + 32 * i;
        const int gr = min(row0 + r, sg.N - 1);
        bulk_g2s_stream(pk + (size_t)st * kPkBytes + (size_t)r * kPkRowBytes,
                        sg.w + (size_t)gr * rowbytes + (size_t)g0 * 32, bytes, &pk_full[st], pol);
      }
    };
    auto issue_b = [&](int g) {  // activations of group g: one 8 KB block in operand layout
      if (lane == 0) {
        const int st = g % kExStages;
        mbar_arrive_expect_tx(&b_full[st], kBBytes);
        bulk_g2s(ex + (size_t)st * (kABytes + kBBytes) + kABytes, p.xq + (size_t)g * kBBytes,
                 kBBytes, &b_full[st]);
      }
    };
    for (int c = 0; c < kPkStages && c < nchunks; ++c) issue_chunk(c);  // weights: no dependency
    pdl_trigger();
    pdl_wait();  // the quantised activations come from the kernel before this one
    constexpr int kAhead = 3;  // activation tiles kept in flight
    for (int g = 0; g < kAhead && g < ngroups; ++g) issue_b(g);
    for (int g = 0; g < ngroups; ++g) {
      const int c = g / kChunkGroups, gi = g % kChunkGroups;
      const int st = g % kExStages;
      // refill the packed ring: chunk c+2 goes where chunk c-1 was, once every expander left it
      if (gi == 0 && c >= 1 && c + kPkStages - 1 < nchunks) {
        ok = mma_wait(ok, &pk_free[(c - 1) % kPkStages], (uint32_t)(((c - 1) / kPkStages) & 1),
                      p.status);
        issue_chunk(c + kPkStages - 1);
      }
      ok = mma_wait(ok, &a_full[st], (uint32_t)((g / kExStages) & 1), p.status);
      ok = mma_wait(ok, &b_full[st], (uint32_t)((g / kExStages) & 1), p.status);
      if (lane == 0) {
        tc_fence_after();
        const uint32_t abase = smem_u32(ex + (size_t)st * (kABytes + kBBytes));
        const uint32_t bbase = abase + kABytes;
#pragma unroll
        for (int j = 0; j < 4; ++j)  // K = 32 bytes per instruction = 2 core matrices
          umma_i8(tmem, umma_desc(abase + j * 256, 128, 1024),
                  umma_desc(bbase + j * 256, 128, 1024), (g > 0 || j > 0) ? 1u : 0u);
        umma_commit(&st_free[st]);  // arrives once these (and all earlier) MMAs read the stage
      }
      __syncwarp();
      // activations kAhead groups ahead, into a stage whose previous MMAs are done
      const int g2 = g + kAhead;
      if (g2 < ngroups) {
        if (g2 >= kExStages)
          ok = mma_wait(ok, &st_free[g2 % kExStages], (uint32_t)(((g2 / kExStages) - 1) & 1),
                        p.status);
        issue_b(g2);
      }
    }
    if (lane == 0) umma_commit(done);
  } else {
    // ================= expander warps ========================================================
    pdl_wait();
    if (tid < kMmaTokens) {
      sd[tid] = p.d[tid];
      ssum[tid] = p.sumq[tid];
    }
    const int erow = tid >> 1, ehalf = tid & 1;
    for (int g = 0; g < ngroups; ++g) {
      const int c = g / kChunkGroups, gi = g % kChunkGroups;
      const int st = g % kExStages;
      if (gi == 0)
        ok = mma_wait(ok, &pk_full[c % kPkStages], (uint32_t)((c / kPkStages) & 1), p.status);
      if (g >= kExStages)  // the MMAs that read this stage four groups ago must be done
        ok = mma_wait(ok, &st_free[st], (uint32_t)(((g / kExStages) - 1) & 1), p.status);
      // this thread's 16 packed bytes (64 weights of one row) -> 4 x 16 bytes of the A operand
      const uint4 w = *reinterpret_cast<const uint4*>(pk + (size_t)(c % kPkStages) * kPkBytes +
                                                      (size_t)erow * kPkRowBytes + gi * 32 +
                                                      ehalf * 16);
      uint8_t* a = ex + (size_t)st * (kABytes + kBBytes) + (size_t)(erow >> 3) * 1024 +
                   (size_t)(erow & 7) * 16;
#pragma unroll
      for (int pl = 0; pl < 4; ++pl) {
        const int sh = 6 - 2 * pl;
        uint4 o;
        o.x = (w.x >> sh) & 0x03030303u;
        o.y = (w.y >> sh) & 0x03030303u;
        o.z = (w.z >> sh) & 0x03030303u;
        o.w = (w.w >> sh) & 0x03030303u;
        // plane pl holds elements 32*pl + j: K bytes 32*pl + 16*half .. +15 = one core-matrix row
        *reinterpret_cast<uint4*>(a + (size_t)(2 * pl + ehalf) * 128) = o;
      }
      fence_proxy_async();  // generic-proxy stores -> visible to the tensor core's async reads
      __syncwarp();
      if (lane == 0) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&a_full[st]))
                     : "memory");
        if (gi == kChunkGroups - 1 || g == ngroups - 1)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(
                           smem_u32(&pk_free[c % kPkStages]))
                       : "memory");
      }
    }
  }
  ok = mma_wait(true, done, 0, p.status) && ok;
  tc_fence_after();

  // ---- epilogue: TMEM lane = weight row, column = token -------------------------------
  if (warp < 4) {
    const int r = warp * 32 + lane;
    const float ws = __ldg(sg.scale);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
      const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(half * 32);
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
          "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
            "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
            "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
            "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
            "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr));
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (r < nrows && ok) {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          const int m = half * 32 + t;
          if (m < p.M) {
            const int total = (int)v[t] - ssum[m];
            const size_t o = (size_t)m * sg.N + row0 + r;
            if (sg.acc) sg.acc[o] = total;
            float y = __fmul_rn(__fmul_rn((float)total, sd[m]), ws);
            if (sg.residual) y = __fadd_rn(y, sg.residual[o]);
            sg.y[o] = y;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kExpWarps)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 64;" ::"r"(tmem));
}

}  // namespace hb

using namespace hb;

// Batched path of hb200_bitlinear_forward_multi (16 <= M <= 64).  Scratch in the context:
// quantised activations in operand layout, their scales and sums.
int hb_bitlinear_mma_run(hb200_ctx* ctx, const hb200_bitlinear_seg* segs, int nseg, int K,
                         const float* d_x, int M, const float* d_rms_gamma, float rms_eps,
                         float* d_act_scale, cudaStream_t st) {
  const size_t xq_bytes = (size_t)(K / 128) * kBBytes;
  HB_REQUIRE(xq_bytes + 1024 <= ctx->scratch_bytes,
             "bitlinear (batched): K=%d needs %zu bytes of activation scratch", K, xq_bytes);
  uint8_t* base = static_cast<uint8_t*>(ctx->d_scratch);
  float* d = reinterpret_cast<float*>(base);
  int32_t* sumq = reinterpret_cast<int32_t*>(base + 256);
  uint8_t* xq = base + 1024;
  QuantParams q = {d_x, d_rms_gamma, rms_eps, K, M, xq, d, sumq, d_act_scale};
  HB_CUDA(launch_pdl(quant_act_kernel, dim3(kMmaTokens), dim3(256), (size_t)K * sizeof(float), st,
                     ctx->pdl, q));
  MmaParams p = {};
  int t = 0;
  for (int s = 0; s < nseg; ++s) {
    p.seg[s] = {static_cast<const uint8_t*>(segs[s].d_packed), segs[s].d_scale,
                segs[s].d_residual, segs[s].d_y, segs[s].d_acc, segs[s].N, t};
    t += (segs[s].N + kMmaRows - 1) / kMmaRows;
  }
  p.nseg = nseg;
  p.K = K;
  p.M = M;
  p.xq = xq;
  p.d = d;
  p.sumq = sumq;
  p.status = ctx->d_status;
  static bool configured = false;
  if (!configured) {
    HB_CUDA(cudaFuncSetAttribute(bitlinear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kMmaSmem));
    configured = true;
  }
  HB_CUDA(launch_pdl(bitlinear_mma_kernel, dim3(t), dim3(kMmaThreads + 32), (size_t)kMmaSmem, st,
                     ctx->pdl, p));
  return HB200_OK;
}
