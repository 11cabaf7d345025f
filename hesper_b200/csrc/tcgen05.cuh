// tcgen05.cuh -- small wrappers shared by the tensor-core kernels: shared-memory matrix
// descriptors, MMA issue / commit / fences, the 2-D tensor-map copy and the run-time lookup
// of the tensor-map encoder.
#pragma once

#include <cuda.h>  // CUtensorMap and its enums only; the encoder comes from the runtime

#include "common.cuh"

namespace hb {

// K-major shared-memory matrix descriptor.  layout 0: no swizzle, core matrices of 8 rows x
// 16 bytes, LBO = byte distance between core matrices adjacent in K, SBO = between 8-row
// groups.  layout 2: 128-byte swizzle, rows of 128 bytes in 1 KB atoms of 8 rows, SBO = 1024.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo,
                                                 uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of this architecture
  d |= (uint64_t)layout << 61;
  return d;
}

// kind::f16 with the A operand in tensor memory (lane = row, two 16-bit K elements per
// 32-bit column) and B through a shared-memory descriptor.
__device__ __forceinline__ void tc_mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

// One box of a 2-D tensor map into shared memory; completion is counted in bytes on `bar`.
// x in elements of the innermost dimension (x * element size must be a multiple of 16).
__device__ __forceinline__ void tc_tma_box_2d(void* dst, const CUtensorMap* tm, int x, int y,
                                              uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Bounded mbarrier wait for kernels whose whole life is microseconds: ~1e5 polls already
// means something is broken.  Once a wait has failed the later ones are skipped, so a broken
// launch ends quickly (and still releases its tensor memory).
__device__ __forceinline__ bool tc_wait(bool ok, uint64_t* bar, uint32_t parity, uint32_t* status) {
  if (!ok) return false;
#pragma unroll 1
  for (uint32_t it = 0; it < (1u << 17); ++it)
    if (mbar_try_wait(bar, parity)) return true;
  atomicOr(status, kStatusMbarTimeout);
  return false;
}

#define HB_TMEM_LD32(v, addr)                                                                  \
  asm volatile(                                                                                \
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                \
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"                                \
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"               \
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),    \
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]),             \
        "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),          \
        "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),          \
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]),          \
        "=r"(v[31])                                                                            \
      : "r"(addr))

#define HB_TMEM_ST32(addr, v)                                                                  \
  asm volatile(                                                                                \
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "                                          \
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"                               \
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(addr),         \
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),  \
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),        \
      "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),      \
      "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]),      \
      "r"(v[29]), "r"(v[30]), "r"(v[31])                                                       \
      : "memory")

typedef CUresult (*TcEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The tensor-map encoder is a driver entry point; it is looked up through the runtime so
// that the library does not link against the driver library.  Null when unavailable.
inline TcEncodeTiledFn tc_tensor_map_encoder() {
  static TcEncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<TcEncodeTiledFn>(f);
  }();
  return fn;
}

}  // namespace hb
