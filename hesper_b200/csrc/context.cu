// context.cu -- context object, error strings and status block of the C ABI.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace hb {

static thread_local char g_err[512] = "no error";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %s (%s) in %s", cudaGetErrorName(e), cudaGetErrorString(e), what);
  // clear the sticky-free error so the next call starts clean
  (void)cudaGetLastError();
  return HB200_ERR_CUDA;
}

}  // namespace hb

int hb_func_smem(hb200_ctx* ctx, const void* func, size_t bytes) {
  for (int i = 0; i < ctx->n_func_smem; ++i) {
    if (ctx->func_smem[i].func == func) {
      if (ctx->func_smem[i].bytes >= bytes) return HB200_OK;
      HB_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
      ctx->func_smem[i].bytes = bytes;
      return HB200_OK;
    }
  }
  HB_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  if (ctx->n_func_smem < 96) ctx->func_smem[ctx->n_func_smem++] = {func, bytes, false};
  return HB200_OK;
}

bool hb_func_flag(hb200_ctx* ctx, const void* func) {
  for (int i = 0; i < ctx->n_func_smem; ++i)
    if (ctx->func_smem[i].func == func) return ctx->func_smem[i].flag;
  return false;
}

void hb_func_set_flag(hb200_ctx* ctx, const void* func) {
  for (int i = 0; i < ctx->n_func_smem; ++i)
    if (ctx->func_smem[i].func == func) ctx->func_smem[i].flag = true;
}

ScratchUse::ScratchUse(hb200_ctx* ctx, cudaStream_t stream) : c(ctx), st(stream) {
  if (c->scratch_depth++ > 0) return;  // an operator inside an operator: the outer scope rules
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  if (cs != cudaStreamCaptureStatusNone) return;
  if (c->scratch_used && c->scratch_stream != st && c->scratch_done != nullptr)
    cudaStreamWaitEvent(st, c->scratch_done, 0);
}

ScratchUse::~ScratchUse() {
  if (--c->scratch_depth > 0) return;
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  if (cs != cudaStreamCaptureStatusNone || c->scratch_done == nullptr) return;
  if (cudaEventRecord(c->scratch_done, st) == cudaSuccess) {
    c->scratch_stream = st;
    c->scratch_used = true;
  } else {
    cudaGetLastError();
  }
}

using namespace hb;

extern "C" const char* hb200_last_error(void) { return g_err; }

extern "C" int hb200_version(void) { return 100; }

// Builds the context object on whatever CUDA context is current on this thread.
static int ctx_build(int device, bool adopted, hb200_ctx** out) {
  cudaDeviceProp prop;
  HB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    set_error("ctx_create: device %d is sm_%d%d; this library is built for sm_100a only", device,
              prop.major, prop.minor);
    return HB200_ERR_UNSUPPORTED;
  }
  hb200_ctx* c = new hb200_ctx();
  c->d_status = nullptr;
  c->d_tickets = nullptr;
  c->d_scratch = nullptr;
  c->device = device;
  c->sm_count = prop.multiProcessorCount;
  c->smem_optin = (int)prop.sharedMemPerBlockOptin;
  c->smem_per_sm = (size_t)prop.sharedMemPerMultiprocessor;
  c->pdl = true;
  c->attn_mode = HB200_ATTN_FAST;
  c->no_mma = false;
  if (const char* e2 = getenv("HB200_NO_MMA")) c->no_mma = e2[0] == '1';
  c->mv_mode = 1;
  if (const char* e3 = getenv("HB200_MV")) c->mv_mode = e3[0] == '0' ? 0 : (e3[0] == '2' ? 2 : 1);
  c->n_func_smem = 0;
  c->attn_cluster_refused = 0;
  c->attn_static_addr = nullptr;
  c->adopted = adopted;
  c->scratch_done = nullptr;
  c->scratch_stream = nullptr;
  c->scratch_used = false;
  c->scratch_depth = 0;
  const char* env = getenv("HB200_NO_PDL");
  if (env && env[0] == '1') c->pdl = false;
  cudaError_t e = cudaMalloc(&c->d_status, 256);
  if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, 256);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_tickets, sizeof(int) * (kCtxTickets + 16));
  if (e == cudaSuccess) e = cudaMemset(c->d_tickets, 0, sizeof(int) * (kCtxTickets + 16));
  c->scratch_bytes = kScratchBytes;
  if (e == cudaSuccess) e = cudaMalloc(&c->d_scratch, c->scratch_bytes);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->scratch_done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    cudaFree(c->d_status);
    cudaFree(c->d_tickets);
    cudaFree(c->d_scratch);
    if (c->scratch_done) cudaEventDestroy(c->scratch_done);
    delete c;
    return cuda_fail(e, "context buffers");
  }
  *out = c;
  return HB200_OK;
}

extern "C" int hb200_ctx_create(int device, hb200_ctx** out) {
  HB_REQUIRE(out != nullptr, "ctx_create: null output pointer");
  *out = nullptr;
  int count = 0;
  HB_CUDA(cudaGetDeviceCount(&count));
  HB_REQUIRE(device >= 0 && device < count, "ctx_create: device %d of %d", device, count);
  HB_CUDA(cudaSetDevice(device));
  return ctx_build(device, false, out);
}

extern "C" int hb200_ctx_create_current(hb200_ctx** out) {
  HB_REQUIRE(out != nullptr, "ctx_create_current: null output pointer");
  *out = nullptr;
  // The caller's context, as the driver API sees it: a host that made its context with
  // cuCtxCreate (native/cuda_bridge.cpp:78-82) has it current on this thread, and the CUDA
  // runtime then works inside it.  No device switch, no primary-context retain.
  typedef int (*cuCtxGetCurrent_t)(void**);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  HB_CUDA(cudaGetDriverEntryPoint("cuCtxGetCurrent", &fn, cudaEnableDefault, &q));
  HB_REQUIRE(fn != nullptr && q == cudaDriverEntryPointSuccess,
             "ctx_create_current: the driver does not export cuCtxGetCurrent");
  void* cur = nullptr;
  const int drc = reinterpret_cast<cuCtxGetCurrent_t>(fn)(&cur);
  HB_REQUIRE(drc == 0 && cur != nullptr,
             "ctx_create_current: no CUDA context is current on this thread (driver code %d)", drc);
  int device = -1;
  HB_CUDA(cudaGetDevice(&device));
  return ctx_build(device, true, out);
}

extern "C" int hb200_ctx_destroy(hb200_ctx* ctx) {
  if (!ctx) return HB200_OK;
  cudaFree(ctx->d_status);
  cudaFree(ctx->d_tickets);
  cudaFree(ctx->d_scratch);
  if (ctx->scratch_done) cudaEventDestroy(ctx->scratch_done);
  delete ctx;
  return HB200_OK;
}

extern "C" int hb200_ctx_sm_count(const hb200_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

extern "C" int hb200_ctx_check(hb200_ctx* ctx, hb200_stream stream, uint32_t* flags) {
  HB_REQUIRE(ctx != nullptr, "ctx_check: null context");
  HB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  uint32_t host[16];
  HB_CUDA(cudaMemcpy(host, ctx->d_status, sizeof(host), cudaMemcpyDeviceToHost));
  if (flags) *flags = host[0];
  if (host[0] != 0) {
    HB_CUDA(cudaMemset(ctx->d_status, 0, 256));
    set_error("device status 0x%x: a bounded wait inside a kernel expired", host[0]);
    return HB200_ERR_TIMEOUT;
  }
  return HB200_OK;
}

extern "C" int hb200_ctx_read_status(hb200_ctx* ctx, hb200_stream stream, uint32_t words[64]) {
  HB_REQUIRE(ctx != nullptr && words != nullptr, "ctx_read_status: null argument");
  HB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  HB_CUDA(cudaMemcpy(words, ctx->d_status, 256, cudaMemcpyDeviceToHost));
  return HB200_OK;
}

extern "C" int hb200_ctx_set_attn_mode(hb200_ctx* ctx, int mode) {
  HB_REQUIRE(ctx != nullptr, "ctx_set_attn_mode: null context");
  HB_REQUIRE(mode >= HB200_ATTN_FAST && mode <= HB200_ATTN_EXACT, "ctx_set_attn_mode: mode %d", mode);
  ctx->attn_mode = mode;
  return HB200_OK;
}
