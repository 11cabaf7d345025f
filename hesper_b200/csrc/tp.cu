// tp.cu -- tensor-parallel exchange step over NVLink: a thin, run-time-loaded binding of
// NCCL.  The reference has no multi-GPU code at all (device 0 is hard-wired,
// Hesper/Backend/CUDA.lean:46); tensor parallelism for the Gemma-shaped model is new work:
// column-split q/k/v/gate/up/LM-head matvecs need no exchange, the row-split o_proj and
// down_proj matvecs end in ONE f32 sum all-reduce of hidden*batch elements each.
//
// NCCL is loaded with dlopen at hb200_tp_init time rather than linked, so the library has
// no NCCL dependency on a single GPU and, inside a process that already carries an NCCL
// (PyTorch), binds to that same copy instead of bringing a second one.
#include <dlfcn.h>
#include <string.h>

#include <cstdlib>

#include "common.cuh"

namespace hb {

typedef struct ncclComm* ncclComm_t;
struct NcclId {
  char internal[128];
};
typedef int (*fn_get_unique_id)(NcclId*);
typedef int (*fn_comm_init_rank)(ncclComm_t*, int, NcclId, int);
typedef int (*fn_all_reduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
typedef int (*fn_comm_destroy)(ncclComm_t);
typedef int (*fn_comm_abort)(ncclComm_t);
typedef int (*fn_async_error)(ncclComm_t, int*);
typedef const char* (*fn_error_string)(int);

struct NcclApi {
  void* handle = nullptr;
  fn_get_unique_id get_unique_id = nullptr;
  fn_comm_init_rank comm_init_rank = nullptr;
  fn_all_reduce all_reduce = nullptr;
  fn_comm_destroy comm_destroy = nullptr;
  fn_comm_abort comm_abort = nullptr;
  fn_async_error async_error = nullptr;
  fn_error_string error_string = nullptr;
};

static NcclApi g_nccl;

static int nccl_load() {
  if (g_nccl.handle) return HB200_OK;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) {
    set_error("tp: cannot load NCCL (libnccl.so.2): %s", dlerror());
    return HB200_ERR_UNSUPPORTED;
  }
  NcclApi a;
  a.handle = h;
  a.get_unique_id = (fn_get_unique_id)dlsym(h, "ncclGetUniqueId");
  a.comm_init_rank = (fn_comm_init_rank)dlsym(h, "ncclCommInitRank");
  a.all_reduce = (fn_all_reduce)dlsym(h, "ncclAllReduce");
  a.comm_destroy = (fn_comm_destroy)dlsym(h, "ncclCommDestroy");
  a.comm_abort = (fn_comm_abort)dlsym(h, "ncclCommAbort");
  a.async_error = (fn_async_error)dlsym(h, "ncclCommGetAsyncError");
  a.error_string = (fn_error_string)dlsym(h, "ncclGetErrorString");
  if (!a.get_unique_id || !a.comm_init_rank || !a.all_reduce || !a.comm_destroy ||
      !a.error_string) {
    set_error("tp: the loaded NCCL lacks a required symbol");
    return HB200_ERR_UNSUPPORTED;
  }
  g_nccl = a;
  return HB200_OK;
}

static int nccl_fail(int r, const char* what) {
  set_error("NCCL error %d (%s) in %s", r, g_nccl.error_string ? g_nccl.error_string(r) : "?", what);
  return HB200_ERR_CUDA;
}

constexpr int kNcclSum = 0, kNcclMax = 2, kNcclUint64 = 5, kNcclFloat32 = 7;

// ---- one-shot all-reduce over peer memory ----------------------------------------------
//
// The exchanges of tensor-parallel decode are tiny (hidden x batch floats: 10 KB at batch 1)
// and there are 84 of them per token, so their cost is latency, not bandwidth.  Every rank
// owns an exchange buffer that all peers map (CUDA IPC); an all-reduce is ONE kernel:
//   push   each CTA stores its chunk of the input into slot [epoch][my rank] of EVERY
//          rank's buffer (plain peer stores over NVLink), fences, then writes the call's
//          sequence number into flag [epoch][my rank][cta] on every rank;
//   wait   the CTA polls its own W flags (its own memory) until they carry the number;
//   reduce it adds the W slots in rank order -- the same order on every rank, so all ranks
//          hold bit-identical results -- and writes the chunk back.
// Two epochs alternate, so a rank that runs ahead never overwrites a slot a slower peer is
// still reading (it cannot be two calls ahead: the call in between needs that peer's flags).
// The sequence number lives in device memory and is advanced by the kernel itself, so a
// captured graph replays correctly.  Every wait is bounded; on expiry the kernel raises the
// status flag and returns.  No multicast, no NVLS: plain loads and stores.
constexpr int kPeerMaxRanks = 8;
constexpr int kPeerMaxCtas = 64;
constexpr size_t kPeerSlotBytes = (size_t)2560 * 64 * 4;  // hidden 2560 x 64 tokens of f32
// one flag per 128-byte line: the CTAs of a launch poll and are written to concurrently, and
// flags sharing a line made every poll contend with the incoming remote stores
constexpr int kPeerFlagStride = 32;
constexpr size_t kPeerFlagBytes =
    (size_t)2 * kPeerMaxRanks * kPeerMaxCtas * kPeerFlagStride * sizeof(uint32_t);
// A second region of the same shape for the flag-in-data exchange below: every 8-byte word
// is {f32 value, u32 sequence number}, so it holds half as many values per slot.
constexpr size_t kPeerLLBase = 2 * kPeerMaxRanks * kPeerSlotBytes + kPeerFlagBytes;
constexpr int kPeerLLMaxTokens = 256;
constexpr size_t kPeerLLSlotBytes = (size_t)2560 * kPeerLLMaxTokens * 8;  // 5 MB per (epoch, rank)
constexpr size_t kPeerBufBytes = kPeerLLBase + 2 * kPeerMaxRanks * kPeerLLSlotBytes;

// Bounded waits: a poll loop looks at the nanosecond timer every 256 polls and gives up
// `timeout_ns` after it started (default one second, hb200_tp_set_timeout_ms changes it).
__device__ __forceinline__ unsigned long long tp_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
struct Deadline {
  unsigned long long end;
  uint32_t polls;
  __device__ __forceinline__ explicit Deadline(unsigned long long timeout_ns)
      : end(tp_now_ns() + timeout_ns), polls(0) {}
  __device__ __forceinline__ bool expired() {
    return ((++polls & 255u) == 0u) && tp_now_ns() > end;
  }
};

struct PeerParams {
  unsigned long long timeout_ns;
  unsigned char* buf[kPeerMaxRanks];  // every rank's exchange buffer (own one included)
  void* io;                           // local vector, reduced in place
  size_t n;                           // elements
  int rank, nranks;
  uint32_t* seq;                      // [0] last finished call, [1] finishing ticket
  uint32_t* status;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// T = float with sum, or unsigned long long with max.  Elements are moved as 16-byte words.
template <typename T, bool kMax>
__global__ void __launch_bounds__(256) peer_allreduce_kernel(const __grid_constant__ PeerParams p) {
  pdl_trigger();
  pdl_wait();
  constexpr int kPer16 = 16 / (int)sizeof(T);
  const int tid = threadIdx.x, cta = blockIdx.x, W = p.nranks;
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(p.seq) + 1u;
  const int epoch = (int)(seq & 1u);
  const size_t nvec = (p.n + kPer16 - 1) / kPer16;             // 16-byte words (buffers are padded)
  const size_t per = (nvec + gridDim.x - 1) / gridDim.x;
  const size_t v0 = (size_t)cta * per, v1 = v0 + per < nvec ? v0 + per : nvec;
  uint4* io = reinterpret_cast<uint4*>(p.io);
  const size_t slot_off = ((size_t)epoch * kPeerMaxRanks + p.rank) * kPeerSlotBytes;
  // ---- push -------------------------------------------------------------------------
  for (size_t v = v0 + tid; v < v1; v += 256) {
    const uint4 x = io[v];
    for (int r = 0; r < W; ++r) reinterpret_cast<uint4*>(p.buf[r] + slot_off)[v] = x;
  }
  // the barrier orders every thread's pushes before the flag writers' fence + release store
  // (cumulative at system scope), so one fence per flag writer is enough
  __syncthreads();
  const size_t flag_base = 2 * kPeerMaxRanks * kPeerSlotBytes;
  if (tid < W) {
    uint32_t* f = reinterpret_cast<uint32_t*>(p.buf[tid] + flag_base) +
                  (((size_t)epoch * kPeerMaxRanks + p.rank) * kPeerMaxCtas + cta) * kPeerFlagStride;
    __threadfence_system();
    st_release_sys(f, seq);
  }
  // ---- wait for every rank's chunk (flags in this rank's own buffer) ------------------------
  __shared__ int s_ok;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < W) {
    const uint32_t* f = reinterpret_cast<const uint32_t*>(p.buf[p.rank] + flag_base) +
                        (((size_t)epoch * kPeerMaxRanks + tid) * kPeerMaxCtas + cta) * kPeerFlagStride;
    bool got = false;
    // once a wait has run out the context is in error: later exchanges look once and go on
    const bool dead = (*reinterpret_cast<volatile uint32_t*>(p.status) & kStatusMbarTimeout) != 0;
    Deadline dl(p.timeout_ns);
#pragma unroll 1
    for (;;) {
      if (ld_acquire_sys(f) == seq) {
        got = true;
        break;
      }
      if (dead || dl.expired()) break;
    }
    if (!got) {
      s_ok = 0;
      atomicOr(p.status, kStatusMbarTimeout);
    }
  }
  __syncthreads();
  // ---- reduce in rank order -----------------------------------------------------------
  if (s_ok) {
    const unsigned char* mine = p.buf[p.rank] + (size_t)epoch * kPeerMaxRanks * kPeerSlotBytes;
    for (size_t v = v0 + tid; v < v1; v += 256) {
      uint4 a = __ldcg(reinterpret_cast<const uint4*>(mine) + v);
      T* av = reinterpret_cast<T*>(&a);
      for (int r = 1; r < W; ++r) {
        const uint4 b = __ldcg(reinterpret_cast<const uint4*>(mine + (size_t)r * kPeerSlotBytes) + v);
        const T* bv = reinterpret_cast<const T*>(&b);
#pragma unroll
        for (int i = 0; i < kPer16; ++i) {
          if (kMax)
            av[i] = bv[i] > av[i] ? bv[i] : av[i];
          else
            av[i] = av[i] + bv[i];
        }
      }
      io[v] = a;
    }
  }
  // ---- the last CTA to finish advances the sequence number -----------------------------
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(&p.seq[1], 1u);
    if (t == gridDim.x - 1) {
      p.seq[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq) = seq;
    }
  }
}

// The same exchange with the RMSNorm that follows it in the decode loop folded in: one CTA
// per token pushes the token's row of partial sums, waits, adds the W rows in rank order
// (bit-identical to the plain all-reduce) and writes y = add + RMSNorm(sum) * gamma with the
// arithmetic of the stand-alone RMSNorm kernel (f64 sum of squares in the same order).
struct PeerNormParams {
  unsigned long long timeout_ns;
  int tok_per_rank;  // two-shot exchange: tokens [r*tok_per_rank, (r+1)*tok_per_rank) belong to rank r
  unsigned char* buf[kPeerMaxRanks];
  const float* x;      // [M][K] this rank's partial sums
  const float* gamma;  // [K]
  const float* add;    // nullable [M][K]
  float* y;            // [M][K]
  float eps;
  int K, rank, nranks;
  uint32_t* seq;
  uint32_t* status;
};

__global__ void __launch_bounds__(256) peer_allreduce_rmsnorm_kernel(
    const __grid_constant__ PeerNormParams p) {
  extern __shared__ __align__(16) float row[];  // [K] the reduced row
  __shared__ double red[8];
  __shared__ int s_ok;
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, m = blockIdx.x, W = p.nranks;
  const int K = p.K, nvec = K >> 2;
  // Rows of up to 3 float4 per thread (K <= 3072) never leave the registers, and every load
  // that does not depend on the exchange is issued before the wait it can hide behind: the
  // norm weights (constants of the model) before the wait on the previous kernel, the
  // addend before the poll for the peers' flags.
  constexpr int kH = 3;
  const bool held = nvec <= kH * 256;
  float4 g4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    g4[j] = (held && v < nvec) ? __ldg(reinterpret_cast<const float4*>(p.gamma) + v)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(p.seq) + 1u;
  const int epoch = (int)(seq & 1u);
  const size_t slot_off = ((size_t)epoch * kPeerMaxRanks + p.rank) * kPeerSlotBytes;
  const uint4* xin = reinterpret_cast<const uint4*>(p.x + (size_t)m * K);
  for (int v = tid; v < nvec; v += 256) {
    const uint4 x = xin[v];
    for (int r = 0; r < W; ++r)
      reinterpret_cast<uint4*>(p.buf[r] + slot_off + (size_t)m * K * 4)[v] = x;
  }
  float4 a4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    a4[j] = (held && p.add && v < nvec)
                ? reinterpret_cast<const float4*>(p.add + (size_t)m * K)[v]
                : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (tid == 0) s_ok = 1;
  // the barrier orders every thread's pushes before the flag writers' release stores below
  // (release at system scope is cumulative over what happened before it in this CTA)
  __syncthreads();
  const size_t flag_base = 2 * kPeerMaxRanks * kPeerSlotBytes;
  if (tid < W) {
    uint32_t* f = reinterpret_cast<uint32_t*>(p.buf[tid] + flag_base) +
                  (((size_t)epoch * kPeerMaxRanks + p.rank) * kPeerMaxCtas + m) * kPeerFlagStride;
    __threadfence_system();
    st_release_sys(f, seq);
    const uint32_t* g = reinterpret_cast<const uint32_t*>(p.buf[p.rank] + flag_base) +
                        (((size_t)epoch * kPeerMaxRanks + tid) * kPeerMaxCtas + m) * kPeerFlagStride;
    bool got = false;
    const bool dead = (*reinterpret_cast<volatile uint32_t*>(p.status) & kStatusMbarTimeout) != 0;
    Deadline dl(p.timeout_ns);
#pragma unroll 1
    for (;;) {
      if (ld_acquire_sys(g) == seq) {
        got = true;
        break;
      }
      if (dead || dl.expired()) break;
    }
    if (!got) {
      s_ok = 0;
      atomicOr(p.status, kStatusMbarTimeout);
    }
  }
  __syncthreads();
  const unsigned char* mine = p.buf[p.rank] + (size_t)epoch * kPeerMaxRanks * kPeerSlotBytes +
                              (size_t)m * K * 4;
  if (s_ok && held) {
    float4 s4[kH];
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      s4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (v < nvec) {
        s4[j] = __ldcg(reinterpret_cast<const float4*>(mine) + v);
        for (int r = 1; r < W; ++r) {  // rank order: the same sum on every rank
          const float4 t =
              __ldcg(reinterpret_cast<const float4*>(mine + (size_t)r * kPeerSlotBytes) + v);
          s4[j].x = __fadd_rn(s4[j].x, t.x);
          s4[j].y = __fadd_rn(s4[j].y, t.y);
          s4[j].z = __fadd_rn(s4[j].z, t.z);
          s4[j].w = __fadd_rn(s4[j].w, t.w);
        }
      }
    }
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < kH; ++j)
      ss += (double)s4[j].x * s4[j].x + (double)s4[j].y * s4[j].y + (double)s4[j].z * s4[j].z +
            (double)s4[j].w * s4[j].w;
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float rinv = (float)(1.0 / sqrt(tot / (double)K + (double)p.eps));
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      if (v >= nvec) continue;
      float4 o;
      o.x = __fmul_rn(__fmul_rn(s4[j].x, rinv), g4[j].x);
      o.y = __fmul_rn(__fmul_rn(s4[j].y, rinv), g4[j].y);
      o.z = __fmul_rn(__fmul_rn(s4[j].z, rinv), g4[j].z);
      o.w = __fmul_rn(__fmul_rn(s4[j].w, rinv), g4[j].w);
      if (p.add) {
        o.x = __fadd_rn(a4[j].x, o.x);
        o.y = __fadd_rn(a4[j].y, o.y);
        o.z = __fadd_rn(a4[j].z, o.z);
        o.w = __fadd_rn(a4[j].w, o.w);
      }
      reinterpret_cast<float4*>(p.y + (size_t)m * K)[v] = o;
    }
  } else if (s_ok) {
    double ss = 0.0;
    for (int k = tid; k < K; k += 256) {
      float a = __ldcg(reinterpret_cast<const float*>(mine) + k);
      for (int r = 1; r < W; ++r)
        a = __fadd_rn(a, __ldcg(reinterpret_cast<const float*>(mine + (size_t)r * kPeerSlotBytes) + k));
      row[k] = a;
      ss += (double)a * a;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    double tot = 0.0;
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float rinv = (float)(1.0 / sqrt(tot / (double)K + (double)p.eps));
    for (int k = tid; k < K; k += 256) {
      float v = __fmul_rn(__fmul_rn(row[k], rinv), p.gamma[k]);
      if (p.add) v = __fadd_rn(p.add[(size_t)m * K + k], v);
      p.y[(size_t)m * K + k] = v;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(&p.seq[1], 1u);
    if (t == gridDim.x - 1) {
      p.seq[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq) = seq;
    }
  }
}

// The fused exchange + RMSNorm again, with the flag carried IN the data (the scheme NCCL calls
// LL): every value travels as one 8-byte store {value, sequence number of this call}, which
// the memory system performs atomically (two of them per 16-byte access), so the receiver needs no separate flag, the sender
// no fence and no wait for its stores to be acknowledged -- one NVLink crossing instead of
// three on the critical path.  Each thread polls exactly the words it will add (bounded), the
// own contribution never leaves the registers, sums are formed in rank order (bit-identical
// on all ranks and to the other exchange paths).  K <= 3072, K % 4 == 0, M * K * 8 bytes
// within a slot (256 tokens of 2560).  A slot is reused every second call and sequence numbers only grow, so a
// stale word can never pass for a fresh one.
// Two {value, flag} words per 16-byte access: each aligned 8-byte half arrives whole.
__device__ __forceinline__ void st_pairs_sys(void* p, float v0, float v1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %2};" ::"l"(p),
               "r"(__float_as_uint(v0)), "r"(flag), "r"(__float_as_uint(v1))
               : "memory");
}
__device__ __forceinline__ bool ld_pairs_sys(const void* p, uint32_t want, float* v0, float* v1) {
  uint32_t a, fa, b, fb;
  asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(a), "=r"(fa), "=r"(b), "=r"(fb)
               : "l"(p)
               : "memory");
  *v0 = __uint_as_float(a);
  *v1 = __uint_as_float(b);
  return fa == want && fb == want;
}

__global__ void __launch_bounds__(256) peer_allreduce_rmsnorm_ll_kernel(
    const __grid_constant__ PeerNormParams p) {
  __shared__ double red[8];
  __shared__ int s_bad;
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, m = blockIdx.x, W = p.nranks;
  const int K = p.K, nvec = K >> 2;
  constexpr int kH = 3;
  float4 g4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    g4[j] = v < nvec ? __ldg(reinterpret_cast<const float4*>(p.gamma) + v)
                     : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (tid == 0) s_bad = 0;
  pdl_wait();
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(p.seq) + 1u;
  const int epoch = (int)(seq & 1u);
  const size_t row_off = (size_t)m * K * 8;
  // ---- push this rank's row to every other rank ---------------------------------------
  float4 x4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    x4[j] = v < nvec ? reinterpret_cast<const float4*>(p.x + (size_t)m * K)[v]
                     : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int r = 0; r < W; ++r) {
    if (r == p.rank) continue;
    unsigned char* dst = p.buf[r] + kPeerLLBase +
                         ((size_t)epoch * kPeerMaxRanks + p.rank) * kPeerLLSlotBytes + row_off;
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      if (v >= nvec) continue;
      unsigned char* d = dst + (size_t)v * 32;
      st_pairs_sys(d, x4[j].x, x4[j].y, seq);
      st_pairs_sys(d + 16, x4[j].z, x4[j].w, seq);
    }
  }
  float4 a4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    a4[j] = (p.add && v < nvec) ? reinterpret_cast<const float4*>(p.add + (size_t)m * K)[v]
                                : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // ---- collect in rank order ------------------------------------------------------------
  float4 s4[kH];
  // once a wait has run out the context is in error: later exchanges do not wait again, so a
  // broken run ends in seconds instead of a second per exchange
  bool ok = (*reinterpret_cast<volatile uint32_t*>(p.status) & kStatusMbarTimeout) == 0;
  Deadline dl(p.timeout_ns);
  for (int r = 0; r < W; ++r) {
    const unsigned char* src = p.buf[p.rank] + kPeerLLBase +
                               ((size_t)epoch * kPeerMaxRanks + r) * kPeerLLSlotBytes + row_off;
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      float4 t = x4[j];
      if (r != p.rank && v < nvec) {
        const unsigned char* q = src + (size_t)v * 32;
        float* tv = reinterpret_cast<float*>(&t);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          bool got = false;
#pragma unroll 1
          while (ok) {
            if (ld_pairs_sys(q + 16 * e, seq, &tv[2 * e], &tv[2 * e + 1])) {
              got = true;
              break;
            }
            if (dl.expired()) break;
          }
          ok = ok && got;
        }
      }
      if (r == 0) {
        s4[j] = t;
      } else {
        s4[j].x = __fadd_rn(s4[j].x, t.x);
        s4[j].y = __fadd_rn(s4[j].y, t.y);
        s4[j].z = __fadd_rn(s4[j].z, t.z);
        s4[j].w = __fadd_rn(s4[j].w, t.w);
      }
    }
  }
  if (!ok) {
    s_bad = 1;
    atomicOr(p.status, kStatusMbarTimeout);
  }
  double ss = 0.0;
#pragma unroll
  for (int j = 0; j < kH; ++j)
    ss += (double)s4[j].x * s4[j].x + (double)s4[j].y * s4[j].y + (double)s4[j].z * s4[j].z +
          (double)s4[j].w * s4[j].w;
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  if (!s_bad) {
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float rinv = (float)(1.0 / sqrt(tot / (double)K + (double)p.eps));
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      if (v >= nvec) continue;
      float4 o;
      o.x = __fmul_rn(__fmul_rn(s4[j].x, rinv), g4[j].x);
      o.y = __fmul_rn(__fmul_rn(s4[j].y, rinv), g4[j].y);
      o.z = __fmul_rn(__fmul_rn(s4[j].z, rinv), g4[j].z);
      o.w = __fmul_rn(__fmul_rn(s4[j].w, rinv), g4[j].w);
      if (p.add) {
        o.x = __fadd_rn(a4[j].x, o.x);
        o.y = __fadd_rn(a4[j].y, o.y);
        o.z = __fadd_rn(a4[j].z, o.z);
        o.w = __fadd_rn(a4[j].w, o.w);
      }
      reinterpret_cast<float4*>(p.y + (size_t)m * K)[v] = o;
    }
  }
  // ---- the last CTA to finish advances the sequence number -----------------------------
  if (tid == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(&p.seq[1], 1u);
    if (t == gridDim.x - 1) {
      p.seq[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq) = seq;
    }
  }
}

// The two-shot form of the same exchange for larger batches (reduce-scatter, then all-gather,
// by TOKEN): rank r owns tokens [r*T, (r+1)*T).  The CTA of a token pushes this rank's partial
// row to the owner only; the owner adds the W rows in rank order, applies the RMSNorm
// (+ residual) -- it holds the whole row -- and pushes the finished row to every peer, whose CTA
// of that token copies it out.  Per rank and exchange 2*n*(W-1)/W values cross NVLink instead
// of the one-shot's n*(W-1), and every rank holds the owner's bits.  Same slots, sequence
// numbers and flag-in-data words as the one-shot kernel: in a rank's buffer the rows it owns
// receive partials (slot of the sender), the other rows receive results (slot of the owner).
__global__ void __launch_bounds__(256) peer_allreduce_rmsnorm_ll2_kernel(
    const __grid_constant__ PeerNormParams p) {
  __shared__ double red[8];
  __shared__ int s_bad;
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, m = blockIdx.x, W = p.nranks;
  const int K = p.K, nvec = K >> 2;
  const int owner = m / p.tok_per_rank;
  constexpr int kH = 3;
  float4 g4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    g4[j] = (owner == p.rank && v < nvec) ? __ldg(reinterpret_cast<const float4*>(p.gamma) + v)
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (tid == 0) s_bad = 0;
  pdl_wait();
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(p.seq) + 1u;
  const int epoch = (int)(seq & 1u);
  const size_t row_off = (size_t)m * K * 8;
  auto slot = [&](int in_rank, int from_rank) {
    return p.buf[in_rank] + kPeerLLBase +
           ((size_t)epoch * kPeerMaxRanks + from_rank) * kPeerLLSlotBytes + row_off;
  };
  bool ok = (*reinterpret_cast<volatile uint32_t*>(p.status) & kStatusMbarTimeout) == 0;
  Deadline dl(p.timeout_ns);
  auto poll = [&](const unsigned char* q, float4& t) {
    float* tv = reinterpret_cast<float*>(&t);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      bool got = false;
#pragma unroll 1
      while (ok) {
        if (ld_pairs_sys(q + 16 * e, seq, &tv[2 * e], &tv[2 * e + 1])) {
          got = true;
          break;
        }
        if (dl.expired()) break;
      }
      ok = ok && got;
    }
  };
  float4 x4[kH];
#pragma unroll
  for (int j = 0; j < kH; ++j) {
    const int v = tid + j * 256;
    x4[j] = v < nvec ? reinterpret_cast<const float4*>(p.x + (size_t)m * K)[v]
                     : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (owner != p.rank) {
    // ---- not mine: partial row to the owner, finished row back from it ---------------------
    unsigned char* dst = slot(owner, p.rank);
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      if (v >= nvec) continue;
      st_pairs_sys(dst + (size_t)v * 32, x4[j].x, x4[j].y, seq);
      st_pairs_sys(dst + (size_t)v * 32 + 16, x4[j].z, x4[j].w, seq);
    }
    const unsigned char* src = slot(p.rank, owner);
    float4 y4[kH];
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      y4[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (v < nvec) poll(src + (size_t)v * 32, y4[j]);
    }
    if (!ok) {
      s_bad = 1;
      atomicOr(p.status, kStatusMbarTimeout);
    }
    __syncthreads();
    if (!s_bad) {
#pragma unroll
      for (int j = 0; j < kH; ++j) {
        const int v = tid + j * 256;
        if (v < nvec) reinterpret_cast<float4*>(p.y + (size_t)m * K)[v] = y4[j];
      }
    }
  } else {
    // ---- mine: collect in rank order, normalise, send the row to everybody -----------------
    float4 a4[kH];
#pragma unroll
    for (int j = 0; j < kH; ++j) {
      const int v = tid + j * 256;
      a4[j] = (p.add && v < nvec) ? reinterpret_cast<const float4*>(p.add + (size_t)m * K)[v]
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float4 s4[kH];
    for (int r = 0; r < W; ++r) {
      const unsigned char* src = slot(p.rank, r);
#pragma unroll
      for (int j = 0; j < kH; ++j) {
        const int v = tid + j * 256;
        float4 t = x4[j];
        if (r != p.rank && v < nvec) poll(src + (size_t)v * 32, t);
        if (r == 0) {
          s4[j] = t;
        } else {
          s4[j].x = __fadd_rn(s4[j].x, t.x);
          s4[j].y = __fadd_rn(s4[j].y, t.y);
          s4[j].z = __fadd_rn(s4[j].z, t.z);
          s4[j].w = __fadd_rn(s4[j].w, t.w);
        }
      }
    }
    if (!ok) {
      s_bad = 1;
      atomicOr(p.status, kStatusMbarTimeout);
    }
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < kH; ++j)
      ss += (double)s4[j].x * s4[j].x + (double)s4[j].y * s4[j].y + (double)s4[j].z * s4[j].z +
            (double)s4[j].w * s4[j].w;
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (!s_bad) {
      double tot = 0.0;
#pragma unroll
      for (int i = 0; i < 8; ++i) tot += red[i];
      const float rinv = (float)(1.0 / sqrt(tot / (double)K + (double)p.eps));
#pragma unroll
      for (int j = 0; j < kH; ++j) {
        const int v = tid + j * 256;
        if (v >= nvec) continue;
        float4 o;
        o.x = __fmul_rn(__fmul_rn(s4[j].x, rinv), g4[j].x);
        o.y = __fmul_rn(__fmul_rn(s4[j].y, rinv), g4[j].y);
        o.z = __fmul_rn(__fmul_rn(s4[j].z, rinv), g4[j].z);
        o.w = __fmul_rn(__fmul_rn(s4[j].w, rinv), g4[j].w);
        if (p.add) {
          o.x = __fadd_rn(a4[j].x, o.x);
          o.y = __fadd_rn(a4[j].y, o.y);
          o.z = __fadd_rn(a4[j].z, o.z);
          o.w = __fadd_rn(a4[j].w, o.w);
        }
        reinterpret_cast<float4*>(p.y + (size_t)m * K)[v] = o;
        for (int r = 0; r < W; ++r) {
          if (r == p.rank) continue;
          unsigned char* d = slot(r, p.rank) + (size_t)v * 32;
          st_pairs_sys(d, o.x, o.y, seq);
          st_pairs_sys(d + 16, o.z, o.w, seq);
        }
      }
    }
  }
  // ---- the last CTA to finish advances the sequence number -----------------------------
  if (tid == 0) {
    __threadfence();
    const uint32_t t = atomicAdd(&p.seq[1], 1u);
    if (t == gridDim.x - 1) {
      p.seq[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.seq) = seq;
    }
  }
}

}  // namespace hb

using namespace hb;

struct hb200_tp {
  ncclComm_t comm;
  int rank, nranks;
  hb200_ctx* ctx;
  unsigned char* peer_buf[kPeerMaxRanks];  // mapped exchange buffers, [rank] is the local one
  bool peer_ready;
  uint32_t* d_seq;   // sequence number and finishing ticket of the peer all-reduce
  float* d_align;    // one float for hb200_tp_align
  unsigned long long timeout_ns;  // bound of every device-side wait of the exchange kernels
  // path selection, read from the environment ONCE at init (same values on every rank: a
  // rank that chose another path than its peers would wait for stores that never come)
  int fuse_max;      // HB200_TP_FUSE_MAX: tokens up to which the fused kernels run
  int two_shot_from; // HB200_TP_TWO_SHOT_FROM: tokens from which the exchange is two-shot
  bool no_ll;        // HB200_TP_NO_LL: flag-after-data kernel instead of flag-in-data
};

// In-place reduction of n elements through the peer buffers, or HB200_ERR_UNSUPPORTED when
// this call does not qualify (not attached, too large, unaligned).
template <typename T, bool kMax>
static int peer_allreduce(hb200_tp* tp, T* d_buf, size_t n, cudaStream_t st) {
  if (!tp->peer_ready || n * sizeof(T) > kPeerSlotBytes || (n * sizeof(T)) % 16 != 0)
    return HB200_ERR_UNSUPPORTED;  // the same answer on every rank: NCCL takes the call
  HB_REQUIRE((reinterpret_cast<uintptr_t>(d_buf) & 15) == 0,
             "tp_allreduce: the buffer must be 16-byte aligned");
  PeerParams p = {};
  for (int r = 0; r < tp->nranks; ++r) p.buf[r] = tp->peer_buf[r];
  p.io = d_buf;
  p.n = n;
  p.rank = tp->rank;
  p.nranks = tp->nranks;
  p.seq = tp->d_seq;
  p.status = tp->ctx->d_status;
  p.timeout_ns = tp->timeout_ns;
  // one CTA per 16 KB, the same count on every rank (it depends on n only)
  size_t ctas = (n * sizeof(T) + 16383) / 16384;
  if (ctas > kPeerMaxCtas) ctas = kPeerMaxCtas;
  if (ctas < 1) ctas = 1;
  HB_CUDA(launch_pdl(peer_allreduce_kernel<T, kMax>, dim3((unsigned)ctas), dim3(256), 0, st,
                     tp->ctx->pdl, p));
  return HB200_OK;
}

extern "C" int hb200_tp_unique_id(unsigned char out[128]) {
  HB_REQUIRE(out != nullptr, "tp_unique_id: null output");
  int rc = nccl_load();
  if (rc) return rc;
  NcclId id;
  int r = g_nccl.get_unique_id(&id);
  if (r != 0) return nccl_fail(r, "ncclGetUniqueId");
  memcpy(out, id.internal, 128);
  return HB200_OK;
}

extern "C" int hb200_tp_init(hb200_ctx* ctx, int rank, int nranks, const unsigned char id[128],
                             hb200_tp** out) {
  HB_REQUIRE(ctx && id && out, "tp_init: null argument");
  HB_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "tp_init: rank %d of %d", rank, nranks);
  *out = nullptr;
  int rc = nccl_load();
  if (rc) return rc;
  if (!ctx->adopted) HB_CUDA(cudaSetDevice(ctx->device));
  NcclId nid;
  memcpy(nid.internal, id, 128);
  ncclComm_t comm = nullptr;
  int r = g_nccl.comm_init_rank(&comm, nranks, nid, rank);
  if (r != 0) return nccl_fail(r, "ncclCommInitRank");
  hb200_tp* tp = new hb200_tp();
  tp->comm = comm;
  tp->rank = rank;
  tp->nranks = nranks;
  tp->ctx = ctx;
  tp->timeout_ns = 1000000000ull;
  const char* e = getenv("HB200_TP_FUSE_MAX");
  tp->fuse_max = e ? atoi(e) : kPeerLLMaxTokens;
  if (tp->fuse_max < 0) tp->fuse_max = 0;
  e = getenv("HB200_TP_TWO_SHOT_FROM");
  tp->two_shot_from = e ? atoi(e) : 33;
  tp->no_ll = getenv("HB200_TP_NO_LL") != nullptr;
  cudaError_t ce = cudaMalloc(reinterpret_cast<void**>(&tp->d_align), sizeof(float));
  if (ce == cudaSuccess) ce = cudaMemset(tp->d_align, 0, sizeof(float));
  if (ce != cudaSuccess) {
    if (g_nccl.comm_destroy) g_nccl.comm_destroy(comm);
    delete tp;
    return cuda_fail(ce, "tp_init: scratch");
  }
  *out = tp;
  return HB200_OK;
}

extern "C" int hb200_tp_set_timeout_ms(hb200_tp* tp, int ms) {
  HB_REQUIRE(tp != nullptr && ms >= 1 && ms <= 60000, "tp_set_timeout_ms: %d ms outside 1..60000", ms);
  tp->timeout_ns = (unsigned long long)ms * 1000000ull;
  return HB200_OK;
}

// Brings the ranks together on the host before a run of bounded waits: one NCCL all-reduce
// of a single float (NCCL's own wait has no deadline, so late ranks are simply waited for),
// then a stream synchronisation.  Host-side work that differs between ranks -- allocation,
// prompt upload, graph capture -- would otherwise eat into the first exchange's deadline.
extern "C" int hb200_tp_align(hb200_tp* tp, hb200_stream stream) {
  if (!tp || tp->nranks == 1) return HB200_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int r = g_nccl.all_reduce(tp->d_align, tp->d_align, 1, kNcclFloat32, kNcclSum, tp->comm, st);
  if (r != 0) return nccl_fail(r, "ncclAllReduce(align)");
  HB_CUDA(cudaStreamSynchronize(st));
  return HB200_OK;
}

extern "C" size_t hb200_tp_peer_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

extern "C" int hb200_tp_peer_export(hb200_tp* tp, unsigned char* out_handle) {
  HB_REQUIRE(tp && out_handle, "tp_peer_export: null argument");
  HB_REQUIRE(tp->nranks <= kPeerMaxRanks, "tp_peer_export: at most %d ranks", kPeerMaxRanks);
  if (!tp->ctx->adopted) HB_CUDA(cudaSetDevice(tp->ctx->device));
  if (!tp->peer_buf[tp->rank]) {
    void* b = nullptr;
    HB_CUDA(cudaMalloc(&b, kPeerBufBytes));
    HB_CUDA(cudaMemset(b, 0, kPeerBufBytes));
    tp->peer_buf[tp->rank] = static_cast<unsigned char*>(b);
    HB_CUDA(cudaMalloc(&tp->d_seq, 2 * sizeof(uint32_t)));
    HB_CUDA(cudaMemset(tp->d_seq, 0, 2 * sizeof(uint32_t)));
    HB_CUDA(cudaDeviceSynchronize());
  }
  cudaIpcMemHandle_t h;
  HB_CUDA(cudaIpcGetMemHandle(&h, tp->peer_buf[tp->rank]));
  memcpy(out_handle, &h, sizeof(h));
  return HB200_OK;
}

extern "C" int hb200_tp_peer_attach(hb200_tp* tp, const unsigned char* all_handles) {
  HB_REQUIRE(tp && all_handles, "tp_peer_attach: null argument");
  HB_REQUIRE(tp->peer_buf[tp->rank] != nullptr, "tp_peer_attach: call hb200_tp_peer_export first");
  if (!tp->ctx->adopted) HB_CUDA(cudaSetDevice(tp->ctx->device));
  for (int r = 0; r < tp->nranks; ++r) {
    if (r == tp->rank || tp->peer_buf[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, all_handles + (size_t)r * sizeof(h), sizeof(h));
    void* ptr = nullptr;
    HB_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    tp->peer_buf[r] = static_cast<unsigned char*>(ptr);
  }
  tp->peer_ready = true;
  return HB200_OK;
}

extern "C" int hb200_tp_peer_attached(const hb200_tp* tp) { return tp && tp->peer_ready ? 1 : 0; }

extern "C" int hb200_tp_destroy(hb200_tp* tp) {
  if (!tp) return HB200_OK;
  for (int r = 0; r < kPeerMaxRanks; ++r) {
    if (!tp->peer_buf[r]) continue;
    if (r == tp->rank)
      cudaFree(tp->peer_buf[r]);
    else
      cudaIpcCloseMemHandle(tp->peer_buf[r]);
  }
  if (tp->d_seq) cudaFree(tp->d_seq);
  if (tp->d_align) cudaFree(tp->d_align);
  if (tp->comm && g_nccl.comm_destroy) g_nccl.comm_destroy(tp->comm);
  delete tp;
  return HB200_OK;
}

extern "C" int hb200_tp_rank(const hb200_tp* tp) { return tp ? tp->rank : 0; }
extern "C" int hb200_tp_size(const hb200_tp* tp) { return tp ? tp->nranks : 1; }

extern "C" int hb200_tp_allreduce_f32(hb200_tp* tp, float* d_buf, size_t n, hb200_stream stream) {
  if (!tp || tp->nranks == 1) return HB200_OK;  // nothing to exchange
  HB_REQUIRE(d_buf != nullptr && n >= 1, "tp_allreduce_f32: bad argument");
  const int pr = peer_allreduce<float, false>(tp, d_buf, n, static_cast<cudaStream_t>(stream));
  if (pr != HB200_ERR_UNSUPPORTED) return pr;
  int r = g_nccl.all_reduce(d_buf, d_buf, n, kNcclFloat32, kNcclSum, tp->comm,
                            static_cast<cudaStream_t>(stream));
  if (r != 0) return nccl_fail(r, "ncclAllReduce(f32, sum)");
  return HB200_OK;
}

extern "C" int hb200_tp_allreduce_max_u64(hb200_tp* tp, unsigned long long* d_buf, size_t n,
                                          hb200_stream stream) {
  if (!tp || tp->nranks == 1) return HB200_OK;
  HB_REQUIRE(d_buf != nullptr && n >= 1, "tp_allreduce_max_u64: bad argument");
  const int pr = peer_allreduce<unsigned long long, true>(tp, d_buf, n,
                                                          static_cast<cudaStream_t>(stream));
  if (pr != HB200_ERR_UNSUPPORTED) return pr;
  int r = g_nccl.all_reduce(d_buf, d_buf, n, kNcclUint64, kNcclMax, tp->comm,
                            static_cast<cudaStream_t>(stream));
  if (r != 0) return nccl_fail(r, "ncclAllReduce(u64, max)");
  return HB200_OK;
}

extern "C" int hb200_tp_allreduce_rmsnorm(hb200_tp* tp, hb200_ctx* ctx, float* d_x,
                                          const float* d_gamma, const float* d_add, float eps,
                                          int M, int K, float* d_y, hb200_stream stream) {
  HB_REQUIRE(ctx && d_x && d_gamma && d_y && M >= 1 && K >= 1, "tp_allreduce_rmsnorm: bad argument");
  if (tp && tp->nranks > 1) {
    // The path is chosen from values that are the same on every rank (M, K, the rank count,
    // whether the peers are attached, the switches read at init): a rank-local fact such as a
    // pointer's alignment is an error, never a reason to take another path than the peers.
    const bool ll = !tp->no_ll && K <= 3072 && M <= kPeerLLMaxTokens &&
                    (size_t)M * K * 8 <= kPeerLLSlotBytes;
    const bool flagged = M <= kPeerMaxCtas && (size_t)M * K * 4 <= kPeerSlotBytes &&
                         (size_t)K * 4 <= 48 * 1024;
    if (tp->peer_ready && M <= tp->fuse_max && K % 4 == 0 && (ll || flagged)) {
      HB_REQUIRE(((reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_gamma) |
                   reinterpret_cast<uintptr_t>(d_add) | reinterpret_cast<uintptr_t>(d_y)) & 15) == 0,
                 "tp_allreduce_rmsnorm: arrays must be 16-byte aligned");
      PeerNormParams p = {};
      for (int r = 0; r < tp->nranks; ++r) p.buf[r] = tp->peer_buf[r];
      p.x = d_x;
      p.gamma = d_gamma;
      p.add = d_add;
      p.y = d_y;
      p.eps = eps;
      p.K = K;
      p.rank = tp->rank;
      p.nranks = tp->nranks;
      p.seq = tp->d_seq;
      p.status = ctx->d_status;
      p.timeout_ns = tp->timeout_ns;
      p.tok_per_rank = (M + tp->nranks - 1) / tp->nranks;
      const bool two_shot = ll && M >= tp->two_shot_from && M >= tp->nranks;
      if (two_shot)
        HB_CUDA(launch_pdl(peer_allreduce_rmsnorm_ll2_kernel, dim3(M), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), ctx->pdl, p));
      else if (ll)
        HB_CUDA(launch_pdl(peer_allreduce_rmsnorm_ll_kernel, dim3(M), dim3(256), 0,
                           static_cast<cudaStream_t>(stream), ctx->pdl, p));
      else
        HB_CUDA(launch_pdl(peer_allreduce_rmsnorm_kernel, dim3(M), dim3(256), (size_t)K * 4,
                           static_cast<cudaStream_t>(stream), ctx->pdl, p));
      return HB200_OK;
    }
    const int rc = hb200_tp_allreduce_f32(tp, d_x, (size_t)M * K, stream);
    if (rc != HB200_OK) return rc;
  }
  return hb200_rmsnorm(ctx, d_x, d_gamma, d_add, eps, M, K, d_y, stream);
}

// Host-side health check of the communicator: 0 = healthy.  A peer that died or never
// joined surfaces here (or as an error of the next collective), never as a device fault.
extern "C" int hb200_tp_check(hb200_tp* tp) {
  if (!tp || tp->nranks == 1 || !g_nccl.async_error) return HB200_OK;
  int async = 0;
  int r = g_nccl.async_error(tp->comm, &async);
  if (r != 0) return nccl_fail(r, "ncclCommGetAsyncError");
  if (async != 0) return nccl_fail(async, "asynchronous communicator state");
  return HB200_OK;
}
