// placeholder until the k-quant kernels land
#include "common.cuh"
using namespace hb;
extern "C" int hb200_kquant_forward(hb200_ctx*, int, const void*, int, int, const float*, int,
                                    const float*, float, const float*, float*, hb200_stream) {
  set_error("kquant: not built yet");
  return HB200_ERR_UNSUPPORTED;
}
extern "C" int hb200_kquant_forward_multi(hb200_ctx*, int, const hb200_kquant_seg*, int, int,
                                          const float*, int, const float*, float, hb200_stream) {
  set_error("kquant: not built yet");
  return HB200_ERR_UNSUPPORTED;
}
extern "C" int hb200_kquant_gateup_gelu(hb200_ctx*, int, const void*, const void*, int, int,
                                        const float*, int, const float*, float, float*,
                                        hb200_stream) {
  set_error("kquant: not built yet");
  return HB200_ERR_UNSUPPORTED;
}
