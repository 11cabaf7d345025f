// common.cuh -- sm_100a building blocks shared by the kernels: bulk (TMA) copies
// completed on mbarriers with bounded waits, programmatic dependent launch,
// mixed-sign dp4a, warp reductions, and the host-side context / error plumbing.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hesper_b200.h"

namespace hb {

constexpr int kWarp = 32;

// Device status block (one per context): word 0 is OR-ed with a kernel-specific
// bit when a bounded wait gives up; word 1 keeps the id of the first reporter.
constexpr uint32_t kStatusMbarTimeout = 1u;
constexpr uint32_t kStatusFlagTimeout = 2u;
constexpr int kCtxTickets = 4096;  // arrival counters kept by a context

// ---- PTX wrappers -----------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Makes mbarrier initialisation visible to the async (TMA) proxy.
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Same, but the warp may stay suspended for up to `ns` nanoseconds per try: for waits that sit
// beside another kernel's compute on the same SM and must not take its issue slots.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_quiet(uint64_t* bar, uint32_t parity, uint32_t* status) {
#pragma unroll 1
  for (uint32_t it = 0; it < (1u << 16); ++it) {  // 2^16 tries of up to 20 us each
    if (mbar_try_wait_suspend(bar, parity, 20000u)) return true;
  }
  if (status) atomicOr(status, kStatusMbarTimeout);
  return false;
}

// Bounded wait: each try_wait already blocks for a hardware time slice, so the
// cap below is seconds of wall time, far beyond any legitimate copy.  On expiry
// the status word is set and the caller carries on (results are then invalid
// but the kernel terminates and the context stays usable).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* status) {
#pragma unroll 1
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  if (status) atomicOr(status, kStatusMbarTimeout);
  return false;
}

// 1-D bulk copy global -> shared through the TMA unit; completion is counted in
// bytes on `bar`.  dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Same with an L2 evict-first hint: weights are streamed once per token.
__device__ __forceinline__ void bulk_g2s_stream(void* dst, const void* src, uint32_t bytes,
                                                uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Programmatic dependent launch: `pdl_wait` blocks until the kernels this one
// depends on have completed and their writes are visible; `pdl_trigger` lets
// the next kernel in the stream start its independent prologue (weight
// prefetch).  Both are no-ops when the launch carries no such dependency.
// Rule for every kernel launched this way: a buffer that an earlier kernel of the chain writes
// (activations, residual streams) is never read through the read-only path (__ldg /
// ld.global.nc) -- this kernel is resident while its predecessor still runs on the same SM, the
// predecessor's own loads can leave lines of that buffer in L1, and the read-only path may
// return them after the wait.  Such buffers are read with __ldcg (ld.global.cg, L2) or plain
// loads; __ldg is for weights, scales and norm weights only.  Seen once: a two-launches-per-SM
// matvec that read the hidden state with __ldg lost token parity on a 2-layer model while every
// single-operator test stayed bit-exact.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Four u8 x four s8 products added to c.
__device__ __forceinline__ int dp4a_us(uint32_t a_u8, uint32_t b_s8, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_s8), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a_u8, uint32_t b_u8, int c) {
  int d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8), "r"(b_u8), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a_s8, uint32_t b_s8, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8), "r"(b_s8), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a_s8, uint32_t b_u8, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_s8), "r"(b_u8), "r"(c));
  return d;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- host side ----------------------------------------------------------------

void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define HB_CUDA(expr)                                        \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) return hb::cuda_fail(_e, #expr);  \
  } while (0)

#define HB_REQUIRE(cond, ...)        \
  do {                               \
    if (!(cond)) {                   \
      hb::set_error(__VA_ARGS__);    \
      return HB200_ERR_INVALID;      \
    }                                \
  } while (0)

// Launch with the programmatic-stream-serialisation attribute so consecutive
// kernels of a decode step overlap their weight prefetch with the predecessor.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace hb

// batched (16..64 token) ternary path on the tensor cores, bitlinear_mma.cu
int hb_bitlinear_mma_run(struct hb200_ctx* ctx, const hb200_bitlinear_seg* segs, int nseg, int K,
                         const float* d_x, int M, const float* d_rms_gamma, float rms_eps,
                         float* d_act_scale, cudaStream_t st);

// batched (16..64 token) LM head on the tensor cores, lmhead_mma.cu
int hb_lmhead_mma_run(struct hb200_ctx* ctx, const void* d_table, int dtype, long V, int K,
                      const float* d_x, int M, const float* d_rms_gamma, float rms_eps,
                      float* d_logits, unsigned long long* d_keys, cudaStream_t st);

// Layout of the context's device scratch (one stream at a time uses it; regions of ops that
// never overlap in time may overlap in space):
constexpr size_t kScratchBytes = (size_t)24 << 20;
constexpr size_t kScratchActs = 0;                     // batched ternary: d[64], sumq[64], int8 tiles
constexpr size_t kScratchGlu = (size_t)2 << 20;       // batched gate/up products before the GLU
constexpr size_t kScratchLmSplit = (size_t)8 << 20;   // 16-bit products: hi/lo activation tiles
constexpr size_t kScratchRowScale = ((size_t)16 << 20) - 4096;  // f16 products: one power-of-two
                                                       // scale per staged activation row
constexpr size_t kScratchSplitK = (size_t)16 << 20;   // batched paths: split-K partials

// the two halves of it, also used by the batched k-quant path (weights dequantised to f16)
int hb_gemm16_split(struct hb200_ctx* ctx, int dtype, int K, const float* d_x, int M,
                    const float* d_rms_gamma, float rms_eps, int single, cudaStream_t st);
int hb_gemm16_split_pre(struct hb200_ctx* ctx, int dtype, int K, const float* d_x, int M,
                        const float* d_pre_base, const float* d_pre_gamma, float* d_pre_out,
                        const float* d_rms_gamma, float rms_eps, int single, cudaStream_t st);
int hb_gemm16_mma(struct hb200_ctx* ctx, const void* d_table, int dtype, long V, int K, int M,
                  float* d_y, const float* d_residual, long ldy, unsigned long long* d_keys,
                  int table_constant, cudaStream_t st);
// batched Q4_K with the dequantiser fused into the tensor-core kernel, kquant_mma.cu
struct HbKqSeg {
  const uint8_t* blocks;
  long N;
  float* y;
  const float* residual;
  long ldy;
  int glu;
};
int hb_kq_mma_run_multi(struct hb200_ctx* ctx, const HbKqSeg* segs, int nseg, int K, int M,
                        int NT, cudaStream_t st, int fmt = HB200_FMT_Q4_K);
int hb_kq_mma_run(struct hb200_ctx* ctx, const uint8_t* d_blocks, int K, long N, int M, int NT,
                  float* d_y, const float* d_residual, long ldy, int glu, cudaStream_t st,
                  int fmt = HB200_FMT_Q4_K);

struct hb200_ctx {
  int device;
  int sm_count;
  int smem_optin;      // max dynamic shared memory per block
  uint32_t* d_status;  // 64 words
  int* d_tickets;      // kCtxTickets zero-initialised arrival counters
  void* d_scratch;     // batched paths: quantised activations, gate/up temporaries
  size_t scratch_bytes;
  bool pdl;            // use programmatic dependent launch
  int attn_mode;       // HB200_ATTN_FAST / PRECISE / EXACT
  bool no_mma;         // HB200_NO_MMA=1: keep batched ternary products on the dp4a kernel
  int mv_mode;         // HB200_MV: 0 never the tensor-core matvec, 1 where it measured faster, 2 wherever it fits
  size_t smem_per_sm;  // shared memory of one SM (two co-resident launches must fit in it)
  // dynamic shared memory already granted to each kernel in this context's CUDA context
  // (the attribute is per device and per context, so it cannot live in a process-wide static)
  struct FuncSmem {
    const void* func;
    size_t bytes;
    bool flag;  // kernel-specific: non-portable cluster sizes already allowed
  } func_smem[96];
  int n_func_smem;
  // The scratch and the arrival counters serve one stream at a time: ScratchUse
  // orders a call behind the previous user when it arrives on another stream.
  cudaEvent_t scratch_done;     // end of the last use outside a stream capture
  cudaStream_t scratch_stream;  // the stream that use was on (never dereferenced: compared only)
  bool scratch_used;
  int scratch_depth;            // nesting of ScratchUse on the calling thread
  uint32_t attn_cluster_refused;  // bit n: the driver refused a cluster of n attention CTAs
  void* attn_static_addr;         // device address of the built-in attention scratch array here
  bool adopted;                   // lives in the caller's own CUDA context: never switch devices
};

// Raises cudaFuncAttributeMaxDynamicSharedMemorySize of `func` to `bytes` once per context.
int hb_func_smem(struct hb200_ctx* ctx, const void* func, size_t bytes);
bool hb_func_flag(struct hb200_ctx* ctx, const void* func);
void hb_func_set_flag(struct hb200_ctx* ctx, const void* func);

// causal attention of a prompt chunk tiled over queries (attention_prefill.cu); 1 = not covered
int hb_attn_prefill_tiled(struct hb200_ctx* ctx, const void* d_q, int q_is_f16, const void* d_k,
                          const void* d_v, const int32_t* d_seqlens, int nseq, int T, int H,
                          int Hkv, int D, int slots, int window, int ring, float scale,
                          void* d_ws, size_t ws_bytes, float* d_out, cudaStream_t st);
size_t hb_attn_prefill_tiled_ws(const struct hb200_ctx* ctx, int nseq, int T, int H, int Hkv, int D,
                                int slots);

// Scope of one operator call that touches the context's scratch or arrival counters.
// Entering on another stream than the previous user's makes this stream wait for the event
// recorded at the end of that use; leaving records the event.  Inside a stream capture nothing
// is recorded or waited for (an event from outside cannot enter a capture): graphs that share a
// context are ordered by whoever replays them.
struct ScratchUse {
  struct hb200_ctx* c;
  cudaStream_t st;
  ScratchUse(struct hb200_ctx* ctx, cudaStream_t stream);
  ~ScratchUse();
  ScratchUse(const ScratchUse&) = delete;
  ScratchUse& operator=(const ScratchUse&) = delete;
};

// one-token ternary matvec on mma.sync (bitlinear_mv.cu); 1 = shape not covered
// rope != nullptr: the three tensors are q, k, v of ONE token; RoPE and the f16 KV-cache write
// run in the kernel's epilogue (q lands rotated in segs[0].d_y, k and v only in the caches)
struct HbRope {
  const double* table;  // [D/2][2] (cos, sin), from hb200_rope_table
  const int32_t* pos;   // [1]
  void* k_cache;        // [Hkv][slots][D] f16 of the token's sequence
  void* v_cache;
  int D, slots, ring;
};
int hb_bl_mv_run(struct hb200_ctx* ctx, const hb200_bitlinear_seg* segs, int nseg, int K, int gu,
                 const float* d_x, const float* gamma, float eps, float* d_act_scale,
                 cudaStream_t st, const HbRope* rope = nullptr);
// one-token Q4_K / Q8_0 matvec on mma.sync (kquant_mv.cu); 1 = shape not covered
int hb_kq_mv_run(struct hb200_ctx* ctx, int fmt, const hb200_kquant_seg* segs, int nseg, int K,
                 int gu, const float* d_x, const float* pre_base, const float* pre_gamma,
                 float* pre_out, const float* gamma, float eps, cudaStream_t st);
