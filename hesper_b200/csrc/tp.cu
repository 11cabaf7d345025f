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

}  // namespace hb

using namespace hb;

struct hb200_tp {
  ncclComm_t comm;
  int rank, nranks;
};

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
  HB_CUDA(cudaSetDevice(ctx->device));
  NcclId nid;
  memcpy(nid.internal, id, 128);
  ncclComm_t comm = nullptr;
  int r = g_nccl.comm_init_rank(&comm, nranks, nid, rank);
  if (r != 0) return nccl_fail(r, "ncclCommInitRank");
  hb200_tp* tp = new hb200_tp{comm, rank, nranks};
  *out = tp;
  return HB200_OK;
}

extern "C" int hb200_tp_destroy(hb200_tp* tp) {
  if (!tp) return HB200_OK;
  if (tp->comm && g_nccl.comm_destroy) g_nccl.comm_destroy(tp->comm);
  delete tp;
  return HB200_OK;
}

extern "C" int hb200_tp_rank(const hb200_tp* tp) { return tp ? tp->rank : 0; }
extern "C" int hb200_tp_size(const hb200_tp* tp) { return tp ? tp->nranks : 1; }

extern "C" int hb200_tp_allreduce_f32(hb200_tp* tp, float* d_buf, size_t n, hb200_stream stream) {
  if (!tp || tp->nranks == 1) return HB200_OK;  // nothing to exchange
  HB_REQUIRE(d_buf != nullptr && n >= 1, "tp_allreduce_f32: bad argument");
  int r = g_nccl.all_reduce(d_buf, d_buf, n, kNcclFloat32, kNcclSum, tp->comm,
                            static_cast<cudaStream_t>(stream));
  if (r != 0) return nccl_fail(r, "ncclAllReduce(f32, sum)");
  return HB200_OK;
}

extern "C" int hb200_tp_allreduce_max_u64(hb200_tp* tp, unsigned long long* d_buf, size_t n,
                                          hb200_stream stream) {
  if (!tp || tp->nranks == 1) return HB200_OK;
  HB_REQUIRE(d_buf != nullptr && n >= 1, "tp_allreduce_max_u64: bad argument");
  int r = g_nccl.all_reduce(d_buf, d_buf, n, kNcclUint64, kNcclMax, tp->comm,
                            static_cast<cudaStream_t>(stream));
  if (r != 0) return nccl_fail(r, "ncclAllReduce(u64, max)");
  return HB200_OK;
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
