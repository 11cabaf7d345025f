// placeholder until the attention kernels land
#include "common.cuh"
using namespace hb;
extern "C" size_t hb200_attn_workspace_bytes(const hb200_ctx*, int, int, int, int, int) { return 0; }
extern "C" int hb200_attn_decode(hb200_ctx*, const void*, int, const void*, const void*,
                                 const int32_t*, int, int, int, int, int, int, float, void*, size_t,
                                 float*, hb200_stream) {
  set_error("attention: not built yet");
  return HB200_ERR_UNSUPPORTED;
}
